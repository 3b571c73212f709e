"""Each part alone, built from its spec, against the plain functions; and a toy mixer with state of
its own, defined here, registered, built and stepped without touching the library's files."""
import pytest
import torch

from helpers import TOL, random_tokens, rel_l2
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def make_ctx(entries, starts, dtype):
    from titan_b200 import kernels as K
    from titan_b200.engine.batch import StepContext, StepLayout
    lay = StepLayout(entries, starts, "cuda")
    return StepContext(lay, K.current_stream(), dtype, torch.device("cuda"), {}, {})


def bind(part, prefix, weights, dtype):
    from titan_b200.weights import held_dtype
    specs = {w.name: w for w in part.weight_specs(prefix)}
    part.bind(lambda rel: weights[prefix + rel].to("cuda", held_dtype(specs[prefix + rel].role, dtype)).contiguous())


def rand_for(part, prefix, seed, std=0.1):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for w in part.weight_specs(prefix):
        t = torch.randn(w.shape, generator=g) * (0.1 if w.role == "vector" else std) + (1.0 if w.role == "vector" else 0.0)
        out[w.name] = t.to(torch.bfloat16).float()
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_and_feed_forward_parts(dtype):
    from titan_b200.config import FeedForwardSpec, NormSpec
    from titan_b200.engine.batch import StepEntry
    from titan_b200.parts import FEED_FORWARDS, NORMS
    H, F, T = 72, 200, 11
    norm = NORMS.build(NormSpec("rmsnorm", H, 2e-4, "n.weight"))
    ffn = FEED_FORWARDS.build(FeedForwardSpec("gated_mlp", H, F, prefix="ff."))
    wn, wf = rand_for(norm, "x.", 1), rand_for(ffn, "x.", 2)
    bind(norm, "x.", wn, DT[dtype])
    bind(ffn, "x.", wf, DT[dtype])
    ctx = make_ctx([StepEntry(0, [0] * T, [])], [0], DT[dtype])
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(3))
    h = norm.forward(x.cuda(), ctx)
    want_h = P.rms_norm(x, wn["x.n.weight"], 2e-4)
    assert h.dtype == DT[dtype] and rel_l2(h.float().cpu(), want_h) < TOL[dtype]
    out = x.clone().cuda()
    ffn.forward(h, ctx, out)
    w = {"mlp." + k.split("ff.")[1]: v for k, v in wf.items()}
    want = x + P.mlp_part(w, "", h.float().cpu())
    assert rel_l2(out.cpu(), want) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,qk_norm,rope", [(None, True, True), (24, False, True), (None, True, False)])
def test_attention_mixer_alone(dtype, window, qk_norm, rope):
    """The mixer with its own cache: a prompt for two sequences, then single tokens; options that the
    test models never use (no head norm, no rotation) are built from the spec too."""
    from titan_b200.cache import SequenceCache
    from titan_b200.config import MixerSpec, NormSpec, PositionSpec
    from titan_b200.engine.batch import StepEntry
    from titan_b200.parts import MIXERS
    H, nh, nkv, hd = 56, 6, 3, 32
    spec = MixerSpec("attention", H, nh, nkv, hd, window=window,
                     qk_norm=NormSpec("rmsnorm", hd, 1e-4, "{}_norm.weight") if qk_norm else None,
                     position=PositionSpec("rope", hd, 5000.0) if rope else PositionSpec("none"), prefix="att.")
    mixer = MIXERS.build(spec)
    w = rand_for(mixer, "", 7, std=0.15)
    bind(mixer, "", w, DT[dtype])
    cache = SequenceCache([mixer.cache_need()], 512, 4, 256, DT[dtype], "cuda")
    lens = [100, 37]
    g = torch.Generator().manual_seed(9)
    xs = [torch.randn(n, H, generator=g).to(torch.bfloat16).float() for n in lens]

    def plain(x):
        T = x.shape[0]
        pos = torch.arange(T)
        q = P.linear(x, w["att.q_proj.weight"]).view(T, nh, hd)
        k = P.linear(x, w["att.k_proj.weight"]).view(T, nkv, hd)
        v = P.linear(x, w["att.v_proj.weight"]).view(T, nkv, hd)
        if qk_norm:
            q, k = P.rms_norm(q, w["att.q_norm.weight"], 1e-4), P.rms_norm(k, w["att.k_norm.weight"], 1e-4)
        if rope:
            q, k = P.rope_neox(q, pos, 5000.0), P.rope_neox(k, pos, 5000.0)
        return P.linear(P.causal_attention(q, k, v, window).reshape(T, nh * hd), w["att.o_proj.weight"])
    want = [plain(x) for x in xs]
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    cut = [80, 30]
    cache.reserve({s: n for s, n in zip(slots, lens)})
    ctx = make_ctx([StepEntry(s, [0] * c, []) for s, c in zip(slots, cut)], [0, 0], DT[dtype])
    h = torch.cat([x[:c] for x, c in zip(xs, cut)]).to(DT[dtype]).cuda()
    out = torch.zeros(sum(cut), H, device="cuda")
    mixer.forward(h, ctx, cache.view_for_layer(0), out)
    got = [[out[:80].cpu()], [out[80:].cpu()]]
    at = list(cut)
    while any(a < n for a, n in zip(at, lens)):
        live = [i for i in range(2) if at[i] < lens[i]]
        ctx = make_ctx([StepEntry(slots[i], [0], []) for i in live], [at[i] for i in live], DT[dtype])
        h = torch.stack([xs[i][at[i]] for i in live]).to(DT[dtype]).cuda()
        out = torch.zeros(len(live), H, device="cuda")
        mixer.forward(h, ctx, cache.view_for_layer(0), out)
        for k, i in enumerate(live):
            got[i].append(out[k:k + 1].cpu())
            at[i] += 1
    for i in range(2):
        assert rel_l2(torch.cat(got[i]), want[i]) < TOL[dtype]


# --------------------------------------------------------------------------- #
# A toy mixer with fixed-size state, a toy architecture around it: all defined here.
# --------------------------------------------------------------------------- #
def toy_parts():
    from titan_b200.cache import CacheNeed
    from titan_b200.parts import MIXERS, Mixer
    from titan_b200.weights import WeightSpec

    class DecayMixer(Mixer):
        """state_t = decay * state_{t-1} + x_t . W^T ; output = state_t (per sequence, fixed size)."""

        capturable = False          # forward reads the layout on the host: steps with this mixer are not captured as graphs

        def __init__(self, spec):
            self.spec, self.decay = spec, spec.option("decay", 0.5)

        def cache_need(self):
            return CacheNeed("state", state_shape=(self.spec.hidden_size,))

        def weight_specs(self, prefix):
            return [WeightSpec(prefix + self.spec.prefix + "w.weight", (self.spec.hidden_size, self.spec.hidden_size))]

        def bind(self, get):
            self.w = get(self.spec.prefix + "w.weight")

        def forward(self, h, ctx, cache, out):
            group, index = cache
            state = group.layer_storage(index)                      # [slots, H] float32
            lay = ctx.layout
            u = h.float() @ self.w.float().t()
            starts, slots = lay.q_start.tolist(), lay.slot_of_seq.tolist()
            for b, slot in enumerate(slots):                        # a sequence's tokens in order
                s = state[slot]
                for t in range(starts[b], starts[b + 1]):
                    s = self.decay * s + u[t]
                    out[t] += s
                state[slot] = s
    MIXERS.register("toy_decay", DecayMixer)

    class DecayMixerOnDevice(DecayMixer):
        """The same mixer with its single-token steps written without the host: the layout's arrays index the state on
        the device, so the engine may capture decode steps with it as CUDA graphs (the default: ``capturable``)."""

        capturable = True

        def forward(self, h, ctx, cache, out):
            lay = ctx.layout
            if not lay.all_single:
                return super().forward(h, ctx, cache, out)         # prompts: the scan over a sequence's tokens, on the host
            group, index = cache
            state = group.layer_storage(index)
            slots = lay.slot_of_seq.long()
            new = self.decay * state[slots] + h.float() @ self.w.float().t()
            state[slots] = new
            out += new
    MIXERS.register("toy_decay_on_device", DecayMixerOnDevice)


class ToyConfig:
    """Layers alternate between the toy mixer and attention; layer 2 runs twice."""

    def __init__(self, d):
        self.d = d

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def to_dict(self):
        return dict(self.d)

    def to_model_spec(self):
        from titan_b200.config import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
        d = self.d
        H = d["width"]
        layers = []
        for i in range(d["depth"]):
            if i % 2 == 0:
                mixer = MixerSpec(d.get("mixer", "toy_decay"), H, prefix="mix.", extra=(("decay", d["decay"]),))
            else:
                mixer = MixerSpec("attention", H, 4, 2, 16, position=PositionSpec("rope", 16, 100.0), prefix="attn.")
            layers.append(LayerSpec(i, "pre_norm", mixer, FeedForwardSpec("gated_mlp", H, d["ff"], prefix="ff."),
                                    NormSpec("rmsnorm", H, 1e-5, "n1.weight"), NormSpec("rmsnorm", H, 1e-5, "n2.weight"), f"blocks.{i}."))
        return ModelSpec("ToyForCausalLM", H, d["vocab"], tuple(layers), tuple(d["order"]),
                         NormSpec("rmsnorm", H, 1e-5, "final.weight"), embedding="embed.weight", lm_head=None)


def toy_plain(d, w, tokens):
    x = w["embed.weight"][torch.tensor(tokens)]
    T, pos = len(tokens), torch.arange(len(tokens))
    for i in d["order"]:
        p = f"blocks.{i}."
        h = P.rms_norm(x, w[p + "n1.weight"], 1e-5)
        if i % 2 == 0:
            u, s, rows = P.linear(h, w[p + "mix.w.weight"]), torch.zeros(d["width"]), []
            for t in range(T):
                s = d["decay"] * s + u[t]
                rows.append(s)
            x = x + torch.stack(rows)
        else:
            q = P.rope_neox(P.linear(h, w[p + "attn.q_proj.weight"]).view(T, 4, 16), pos, 100.0)
            k = P.rope_neox(P.linear(h, w[p + "attn.k_proj.weight"]).view(T, 2, 16), pos, 100.0)
            v = P.linear(h, w[p + "attn.v_proj.weight"]).view(T, 2, 16)
            x = x + P.linear(P.causal_attention(q, k, v).reshape(T, 64), w[p + "attn.o_proj.weight"])
        h = P.rms_norm(x, w[p + "n2.weight"], 1e-5)
        x = x + P.mlp_part({k.replace(p + "ff.", "mlp."): v for k, v in w.items() if k.startswith(p + "ff.")}, "", h)
    return P.linear(P.rms_norm(x, w["final.weight"], 1e-5), w["embed.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_mixer_with_state_registers_builds_and_steps(dtype):
    from titan_b200 import Engine, StepEntry, register_architecture
    from titan_b200.parts import declare_weights
    toy_parts()
    register_architecture("ToyForCausalLM", ToyConfig)
    d = {"architectures": ["ToyForCausalLM"], "width": 48, "depth": 3, "ff": 80, "vocab": 120, "decay": 0.6, "order": [0, 1, 2, 2, 1]}
    cfg = ToyConfig(d)
    g = torch.Generator().manual_seed(4)
    w = {}
    for s in declare_weights(cfg.to_model_spec()):
        t = torch.randn(s.shape, generator=g) * (0.1 if s.role == "vector" else 0.12) + (1.0 if s.role == "vector" else 0.0)
        w[s.name] = t.to(torch.bfloat16)
    e = Engine.from_tensors(cfg, w, dtype=dtype, max_tokens=512, max_slots=3)
    assert len(e.cache.groups) == 2 and len(e.model.cache_needs()) == 5      # one cache per run of the order
    w32 = {k: v.float() for k, v in w.items()}
    reqs = [random_tokens(50, 120, 1), random_tokens(21, 120, 2)]
    want = [toy_plain(d, w32, r) for r in reqs]
    for round_ in range(2):                                                     # slots (and their state) are used again
        slots = [e.alloc_slot(), e.alloc_slot()]
        out = e.step([StepEntry(slots[0], reqs[0][:30], list(range(30))), StepEntry(slots[1], reqs[1][:5], list(range(5)))])
        got = [[out[:30]], [out[30:]]]
        at = [30, 5]
        while any(a < len(r) for a, r in zip(at, reqs)):
            live = [i for i in range(2) if at[i] < len(reqs[i])]
            out = e.step([StepEntry(slots[i], [reqs[i][at[i]]], [0]) for i in live])
            for k, i in enumerate(live):
                got[i].append(out[k:k + 1])
                at[i] += 1
        for i in range(2):
            assert rel_l2(torch.cat(got[i]).cpu(), want[i]) < TOL[dtype]
            e.free_slot(slots[i])
    # through the generation loop: the mixer says that it cannot be captured, so every step runs eagerly
    from titan_b200 import SamplerParams
    prompt = reqs[0][:12]
    made = e.generate([prompt], max_tokens=6, params=SamplerParams.greedy(), stop_tokens=[])[0].tokens
    assert len(made) == 6 and e.graph_launches == 0
    logits = toy_plain(d, w32, prompt + made)
    for j, tok in enumerate(made):
        row = logits[len(prompt) - 1 + j]
        assert tok == int(row.argmax()) or float(row.max() - row[tok]) < 0.05 * float(row.abs().max())


def test_a_toy_mixer_with_state_in_captured_decode_steps():
    """The toy mixer with its decode step written for the device: the engine captures its steps as graphs (state of fixed
    size per sequence, read and written inside the graph through the step's slot indices), two requests of unequal
    length generate greedily, one leaves earlier, and every token is the plain implementation's choice."""
    from titan_b200 import Engine, SamplerParams, register_architecture
    from titan_b200.parts import declare_weights
    toy_parts()
    register_architecture("ToyForCausalLM", ToyConfig)
    d = {"architectures": ["ToyForCausalLM"], "width": 64, "depth": 2, "ff": 96, "vocab": 150, "decay": 0.7, "order": [0, 1, 0],
         "mixer": "toy_decay_on_device"}
    cfg = ToyConfig(d)
    g = torch.Generator().manual_seed(9)
    w = {}
    for s in declare_weights(cfg.to_model_spec()):
        t = torch.randn(s.shape, generator=g) * (0.1 if s.role == "vector" else 0.12) + (1.0 if s.role == "vector" else 0.0)
        w[s.name] = t.to(torch.bfloat16)
    w32 = {k: v.float() for k, v in w.items()}
    e = Engine.from_tensors(cfg, w, dtype="float32", max_tokens=512, max_slots=3)
    prompts = [random_tokens(17, 150, 5), random_tokens(4, 150, 6)]
    from titan_b200 import GenerationRequest
    from titan_b200.engine import generate
    outs = generate(e, [GenerationRequest(list(p), n, SamplerParams.greedy(), (), False) for p, n in zip(prompts, (20, 9))])
    assert e.graph_launches > 0                                          # the steps were replayed from graphs
    for prompt, o, n in zip(prompts, outs, (20, 9)):
        assert len(o.tokens) == n
        logits = toy_plain(d, w32, list(prompt) + o.tokens)
        for j, tok in enumerate(o.tokens):
            row = logits[len(prompt) - 1 + j]
            assert tok == int(row.argmax()) or float(row.max() - row[tok]) < 1e-3 * float(row.abs().max()), (j, tok)
    e.cache.check()


# --------------------------------------------------------------------------- #
# A toy feed-forward with routing and a toy position encoding, again defined here only.
# --------------------------------------------------------------------------- #
def more_toy_parts():
    from titan_b200.parts import FEED_FORWARDS, POSITIONS, FeedForward, PositionEncoding
    from titan_b200.weights import WeightSpec

    class PickOne(FeedForward):
        """Each token goes to the ONE expert whose router score (float32) is largest; an expert is
        down(relu(up(h))).  Which expert a token takes depends on the token alone, so a batch changes nothing."""

        def __init__(self, spec):
            self.spec, self.experts = spec, spec.option("experts", 2)

        def weight_specs(self, prefix):
            s, p = self.spec, prefix + self.spec.prefix
            specs = [WeightSpec(p + "router.weight", (self.experts, s.hidden_size), role="vector")]       # kept in float32
            for e in range(self.experts):
                specs += [WeightSpec(p + f"experts.{e}.up.weight", (s.intermediate_size, s.hidden_size)),
                          WeightSpec(p + f"experts.{e}.down.weight", (s.hidden_size, s.intermediate_size))]
            return specs

        def bind(self, get):
            p = self.spec.prefix
            self.router = get(p + "router.weight")
            self.up = [get(p + f"experts.{e}.up.weight") for e in range(self.experts)]
            self.down = [get(p + f"experts.{e}.down.weight") for e in range(self.experts)]

        def forward(self, h, ctx, out):
            choice = (h.float() @ self.router.t()).argmax(dim=1)          # router logits in float32
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    act = torch.relu(h[rows].float() @ self.up[e].float().t()).to(h.dtype)
                    out[rows] += act.float() @ self.down[e].float().t()
    FEED_FORWARDS.register("toy_pick_one", PickOne)

    class StretchedRotary(PositionEncoding):
        """The rotary angles of position p / stretch: the attention mixer only asks for ``rotary_dim`` and a table."""

        def __init__(self, spec):
            self.spec = spec

        @property
        def rotary_dim(self):
            return self.spec.rotary_dim

        def tables(self, device):
            k = torch.arange(self.spec.rotary_dim // 2, dtype=torch.float64)
            inv = torch.tensor(self.spec.theta, dtype=torch.float64) ** (-2.0 * k / self.spec.rotary_dim) / 4.0
            return {"inv_freq": inv.to(torch.float32).to(device)}
    POSITIONS.register("toy_stretched_rope", StretchedRotary)


class ToyRoutedConfig:
    def __init__(self, d):
        self.d = d

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def to_dict(self):
        return dict(self.d)

    def to_model_spec(self):
        from titan_b200.config import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
        d, H = self.d, self.d["width"]
        layers = []
        for i in range(d["depth"]):
            mixer = MixerSpec("attention", H, 3, 1, 32, position=PositionSpec("toy_stretched_rope", 32, 50.0), prefix="attn.")
            ff = (FeedForwardSpec("toy_pick_one", H, d["ff"], prefix="moe.", extra=(("experts", d["experts"]),)) if i % 2 == 0
                  else FeedForwardSpec("gated_mlp", H, d["ff"], prefix="ff."))
            layers.append(LayerSpec(i, "pre_norm", mixer, ff, NormSpec("rmsnorm", H, 1e-6, "n1.weight"),
                                    NormSpec("rmsnorm", H, 1e-6, "n2.weight"), f"blocks.{i}."))
        return ModelSpec("ToyRoutedForCausalLM", H, d["vocab"], tuple(layers), tuple(range(d["depth"])),
                         NormSpec("rmsnorm", H, 1e-6, "final.weight"), embedding="embed.weight", lm_head="head.weight")


def toy_routed_plain(d, w, tokens, margins):
    """Logits; the gap between the two best router scores of every decision is appended to ``margins``."""
    x = w["embed.weight"][torch.tensor(tokens)]
    T, pos = len(tokens), torch.arange(len(tokens)) / 4.0
    for i in range(d["depth"]):
        p = f"blocks.{i}."
        h = P.rms_norm(x, w[p + "n1.weight"], 1e-6)
        q = P.rope_neox(P.linear(h, w[p + "attn.q_proj.weight"]).view(T, 3, 32), pos, 50.0)
        k = P.rope_neox(P.linear(h, w[p + "attn.k_proj.weight"]).view(T, 1, 32), pos, 50.0)
        v = P.linear(h, w[p + "attn.v_proj.weight"]).view(T, 1, 32)
        x = x + P.linear(P.causal_attention(q, k, v).reshape(T, 96), w[p + "attn.o_proj.weight"])
        h = P.rms_norm(x, w[p + "n2.weight"], 1e-6)
        if i % 2 == 0:
            scores = P.linear(h, w[p + "moe.router.weight"])
            choice = scores.argmax(dim=1)
            top2 = scores.topk(2, dim=1).values
            margins.extend((top2[:, 0] - top2[:, 1]).tolist())
            rows = []
            for t in range(T):
                e = int(choice[t])
                act = torch.relu(P.linear(h[t:t + 1], w[p + f"moe.experts.{e}.up.weight"]))
                rows.append(P.linear(act, w[p + f"moe.experts.{e}.down.weight"])[0])
            x = x + torch.stack(rows)
        else:
            x = x + P.mlp_part({k_.replace(p + "ff.", "mlp."): v_ for k_, v_ in w.items() if k_.startswith(p + "ff.")}, "", h)
    return P.linear(P.rms_norm(x, w["final.weight"], 1e-6), w["head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_routed_feed_forward_and_a_toy_position_encoding(dtype):
    """Registered from outside, built by the registries, stepped by the engine (prompts of unequal
    lengths, then single tokens): no file of the framework knows either part."""
    from titan_b200 import Engine, StepEntry, register_architecture
    from titan_b200.parts import declare_weights
    more_toy_parts()
    register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig)
    d = {"architectures": ["ToyRoutedForCausalLM"], "width": 40, "depth": 3, "ff": 56, "vocab": 90, "experts": 3}
    cfg = ToyRoutedConfig(d)
    reqs = [random_tokens(41, 90, 5), random_tokens(17, 90, 6)]
    # A routing decision is discrete: two scores that nearly tie would flip under bfloat16 rounding and
    # say nothing about the parts.  So take the first seed whose decisions are all clear in float32.
    for seed in range(9, 60):
        g = torch.Generator().manual_seed(seed)
        w = {}
        for s in declare_weights(cfg.to_model_spec()):
            std = 2.0 if "router" in s.name else (0.1 if s.role == "vector" else 0.12)
            t = torch.randn(s.shape, generator=g) * std + (1.0 if s.role == "vector" and "router" not in s.name else 0.0)
            w[s.name] = t.to(torch.bfloat16)
        w32 = {k: v.float() for k, v in w.items()}
        margins = []
        want = [toy_routed_plain(d, w32, r, margins) for r in reqs]
        if min(margins) > 0.5:
            break
    else:
        pytest.fail("no seed gave clear routing decisions")
    e = Engine.from_tensors(cfg, w, dtype=dtype, max_tokens=512, max_slots=3)
    slots = [e.alloc_slot(), e.alloc_slot()]
    out = e.step([StepEntry(slots[0], reqs[0][:33], list(range(33))), StepEntry(slots[1], reqs[1][:9], list(range(9)))])
    got, at = [[out[:33]], [out[33:]]], [33, 9]
    while any(a < len(r) for a, r in zip(at, reqs)):
        live = [i for i in range(2) if at[i] < len(reqs[i])]
        out = e.step([StepEntry(slots[i], [reqs[i][at[i]]], [0]) for i in live])
        for k, i in enumerate(live):
            got[i].append(out[k:k + 1])
            at[i] += 1
    for i in range(2):
        assert rel_l2(torch.cat(got[i]).cpu(), want[i]) < TOL[dtype]
        e.free_slot(slots[i])


# --------------------------------------------------------------------------- #
# A layer that reads another layer's cache: it has a query projection only and attends over the keys and
# values that the named layer wrote.  The architecture is defined here; the package knows nothing of it.
# --------------------------------------------------------------------------- #
class SharedCacheConfig:
    def __init__(self, d):
        self.d = d

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def to_dict(self):
        return dict(self.d)

    def to_model_spec(self):
        from titan_b200.config import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
        d = self.d
        H, nh, nkv, hd = d["width"], d["heads"], d["kv_heads"], d["head"]
        layers = []
        for i in range(3):
            mixer = MixerSpec("attention", H, nh, nkv, hd, qk_norm=NormSpec("rmsnorm", hd, 1e-5, "{}_norm.weight"),
                              position=PositionSpec("rope", hd, 1e4), cache_from=0 if i == 2 else None, prefix="attn.")
            layers.append(LayerSpec(i, "pre_norm", mixer, FeedForwardSpec("gated_mlp", H, d["ff"], prefix="ff."),
                                    NormSpec("rmsnorm", H, 1e-5, "n1.weight"), NormSpec("rmsnorm", H, 1e-5, "n2.weight"), f"blocks.{i}."))
        return ModelSpec("SharedCacheForCausalLM", H, d["vocab"], tuple(layers), (0, 1, 2),
                         NormSpec("rmsnorm", H, 1e-5, "final.weight"), embedding="embed.weight", lm_head=None)


def shared_cache_plain(d, w, tokens):
    nh, nkv, hd = d["heads"], d["kv_heads"], d["head"]
    x = w["embed.weight"][torch.tensor(tokens)]
    T, pos = len(tokens), torch.arange(len(tokens))
    kept = {}
    for i in range(3):
        p = f"blocks.{i}."
        h = P.rms_norm(x, w[p + "n1.weight"], 1e-5)
        q = P.rope_neox(P.rms_norm(P.linear(h, w[p + "attn.q_proj.weight"]).view(T, nh, hd), w[p + "attn.q_norm.weight"], 1e-5), pos, 1e4)
        if i == 2:
            k, v = kept[0]                                   # layer 0's keys and values, as its cache holds them
        else:
            k = P.rope_neox(P.rms_norm(P.linear(h, w[p + "attn.k_proj.weight"]).view(T, nkv, hd), w[p + "attn.k_norm.weight"], 1e-5), pos, 1e4)
            v = P.linear(h, w[p + "attn.v_proj.weight"]).view(T, nkv, hd)
            kept[i] = (k, v)
        x = x + P.linear(P.causal_attention(q, k, v).reshape(T, nh * hd), w[p + "attn.o_proj.weight"])
        h = P.rms_norm(x, w[p + "n2.weight"], 1e-5)
        x = x + P.mlp_part({k_.replace(p + "ff.", "mlp."): v_ for k_, v_ in w.items() if k_.startswith(p + "ff.")}, "", h)
    return P.linear(P.rms_norm(x, w["final.weight"], 1e-5), w["embed.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("head", [16, 64])            # 64: the tensor-core attention kernels in bfloat16
def test_a_layer_that_reads_another_layers_cache(dtype, head):
    from titan_b200 import Engine, StepEntry, register_architecture
    from titan_b200.parts import declare_weights
    register_architecture("SharedCacheForCausalLM", SharedCacheConfig)
    d = {"architectures": ["SharedCacheForCausalLM"], "width": 64, "heads": 4, "kv_heads": 2, "head": head, "ff": 96, "vocab": 150}
    cfg = SharedCacheConfig(d)
    g = torch.Generator().manual_seed(9)
    w = {}
    for s in declare_weights(cfg.to_model_spec()):
        t = torch.randn(s.shape, generator=g) * (0.1 if s.role == "vector" else 0.1) + (1.0 if s.role == "vector" else 0.0)
        w[s.name] = t.to(torch.bfloat16)
    assert "blocks.2.attn.k_proj.weight" not in w and "blocks.2.attn.k_norm.weight" not in w and "blocks.2.attn.q_norm.weight" in w
    e = Engine.from_tensors(cfg, w, dtype=dtype, max_tokens=1024, max_slots=2)
    assert len(e.cache.groups) == 1 and sum(n is not None for n in e.model.cache_needs()) == 2     # two layers own a cache, one borrows
    w32 = {k: v.float() for k, v in w.items()}
    reqs = [random_tokens(150, 150, 1), random_tokens(40, 150, 2)]
    want = [shared_cache_plain(d, w32, r) for r in reqs]
    slots = [e.alloc_slot(), e.alloc_slot()]
    cut = [100, 7]
    out = e.step([StepEntry(slots[i], reqs[i][:cut[i]], list(range(cut[i]))) for i in range(2)])
    got = [[out[:cut[0]]], [out[cut[0]:]]]
    at = list(cut)
    while any(a < len(r) for a, r in zip(at, reqs)):
        live = [i for i in range(2) if at[i] < len(reqs[i])]
        out = e.step([StepEntry(slots[i], [reqs[i][at[i]]], [0]) for i in live])
        for k, i in enumerate(live):
            got[i].append(out[k:k + 1])
            at[i] += 1
    for i in range(2):
        assert rel_l2(torch.cat(got[i]).cpu(), want[i]) < TOL[dtype], i
        e.free_slot(slots[i])


# --------------------------------------------------------------------------- #
# A toy norm (mean-centred, with a bias), defined and registered here only.
# --------------------------------------------------------------------------- #
def toy_norm_part():
    from titan_b200.parts import NORMS, Norm
    from titan_b200.weights import WeightSpec

    class CentredNorm(Norm):
        def __init__(self, spec):
            self.spec = spec

        def weight_specs(self, prefix):
            name = prefix + self.spec.weight
            return [WeightSpec(name, (self.spec.size,), "vector", ("one_plus_normal", 0.1)),
                    WeightSpec(name.replace(".weight", ".bias"), (self.spec.size,), "vector", ("normal", 0.1))]

        def bind(self, get):
            self.weight, self.bias = get(self.spec.weight), get(self.spec.weight.replace(".weight", ".bias"))

        def forward(self, x, ctx, rows=None):
            if rows is not None:
                x = x[rows.long()]
            c = x - x.mean(dim=1, keepdim=True)                                   # float32 throughout
            y = c * torch.rsqrt(c.pow(2).mean(dim=1, keepdim=True) + self.spec.eps) * self.weight + self.bias
            return y.to(ctx.dtype)
    NORMS.register("toy_centred", CentredNorm)


class ToyNormConfig(SharedCacheConfig):
    def to_model_spec(self):
        from titan_b200.config import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
        d, H = self.d, self.d["width"]
        norm = lambda name: NormSpec("toy_centred", H, 1e-4, name)
        layers = [LayerSpec(i, "pre_norm", MixerSpec("attention", H, 2, 1, 32, position=PositionSpec("rope", 32, 1e4), prefix="attn."),
                            FeedForwardSpec("gated_mlp", H, d["ff"], prefix="ff."), norm("n1.weight"), norm("n2.weight"), f"blocks.{i}.")
                  for i in range(2)]
        return ModelSpec("ToyNormForCausalLM", H, d["vocab"], tuple(layers), (0, 1), norm("final.weight"),
                         embedding="embed.weight", lm_head=None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_norm(dtype):
    from titan_b200 import Engine, StepEntry, register_architecture
    from titan_b200.parts import declare_weights
    toy_norm_part()
    register_architecture("ToyNormForCausalLM", ToyNormConfig)
    d = {"architectures": ["ToyNormForCausalLM"], "width": 56, "ff": 72, "vocab": 90}
    cfg = ToyNormConfig(d)
    g = torch.Generator().manual_seed(3)
    w = {}
    for s in declare_weights(cfg.to_model_spec()):
        one = 1.0 if s.name.endswith("weight") and s.role == "vector" else 0.0
        w[s.name] = (torch.randn(s.shape, generator=g) * 0.1 + one).to(torch.bfloat16)

    def norm(x, name):
        c = x - x.mean(dim=1, keepdim=True)
        return c * torch.rsqrt(c.pow(2).mean(dim=1, keepdim=True) + 1e-4) * w32[name] + w32[name.replace(".weight", ".bias")]

    def plain(tokens):
        x = w32["embed.weight"][torch.tensor(tokens)]
        T, pos = len(tokens), torch.arange(len(tokens))
        for i in range(2):
            p = f"blocks.{i}."
            h = norm(x, p + "n1.weight")
            q = P.rope_neox(P.linear(h, w32[p + "attn.q_proj.weight"]).view(T, 2, 32), pos, 1e4)
            k = P.rope_neox(P.linear(h, w32[p + "attn.k_proj.weight"]).view(T, 1, 32), pos, 1e4)
            v = P.linear(h, w32[p + "attn.v_proj.weight"]).view(T, 1, 32)
            x = x + P.linear(P.causal_attention(q, k, v).reshape(T, 64), w32[p + "attn.o_proj.weight"])
            x = x + P.mlp_part({k_.replace(p + "ff.", "mlp."): v_ for k_, v_ in w32.items() if k_.startswith(p + "ff.")}, "", norm(x, p + "n2.weight"))
        return P.linear(norm(x, "final.weight"), w32["embed.weight"])
    e = Engine.from_tensors(cfg, w, dtype=dtype, max_tokens=256, max_slots=1)
    w32 = {k: v.float() for k, v in w.items()}
    toks = random_tokens(40, 90, 5)
    s = e.alloc_slot()
    rows = [e.step([StepEntry(s, toks[:25], list(range(25)))])] + [e.step([StepEntry(s, [t], [0])]) for t in toks[25:]]
    e.free_slot(s)
    assert rel_l2(torch.cat(rows).cpu(), plain(toks)) < TOL[dtype]


# --------------------------------------------------------------------------- #
# A toy arrangement: mixer and feed-forward read the same normed input and both add to the stream.
# --------------------------------------------------------------------------- #
def toy_parallel_block():
    from titan_b200.parts import BLOCKS
    from titan_b200.parts.block import PreNormBlock

    class ParallelBlock(PreNormBlock):
        def parts(self):
            return (self.mixer_norm, self.mixer, self.feed_forward)          # one norm: no weights for a second

        def forward(self, x, ctx, cache):
            h = self.mixer_norm.forward(x, ctx)
            self.mixer.forward(h, ctx, cache, x)
            self.feed_forward.forward(h, ctx, x)
    BLOCKS.register("toy_parallel", ParallelBlock)


class ToyParallelConfig(SharedCacheConfig):
    def to_model_spec(self):
        from titan_b200.config import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
        d, H = self.d, self.d["width"]
        layers = [LayerSpec(i, "toy_parallel" if i == 0 else "pre_norm",
                            MixerSpec("attention", H, 2, 2, 16, position=PositionSpec("rope", 16, 1e4), prefix="attn."),
                            FeedForwardSpec("gated_mlp", H, d["ff"], prefix="ff."), NormSpec("rmsnorm", H, 1e-5, "n1.weight"),
                            NormSpec("rmsnorm", H, 1e-5, "n2.weight"), f"blocks.{i}.") for i in range(2)]
        return ModelSpec("ToyParallelForCausalLM", H, d["vocab"], tuple(layers), (0, 1), NormSpec("rmsnorm", H, 1e-5, "final.weight"),
                         embedding="embed.weight", lm_head=None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_arrangement_of_a_block(dtype):
    from titan_b200 import Engine, StepEntry, register_architecture
    from titan_b200.parts import declare_weights
    toy_parallel_block()
    register_architecture("ToyParallelForCausalLM", ToyParallelConfig)
    d = {"architectures": ["ToyParallelForCausalLM"], "width": 40, "ff": 64, "vocab": 70}
    cfg = ToyParallelConfig(d)
    g = torch.Generator().manual_seed(6)
    w = {}
    for s in declare_weights(cfg.to_model_spec()):
        w[s.name] = (torch.randn(s.shape, generator=g) * 0.1 + (1.0 if s.role == "vector" else 0.0)).to(torch.bfloat16)
    assert "blocks.0.n2.weight" not in w and "blocks.1.n2.weight" in w
    w32 = {k: v.float() for k, v in w.items()}

    def plain(tokens):
        x = w32["embed.weight"][torch.tensor(tokens)]
        T, pos = len(tokens), torch.arange(len(tokens))
        for i in range(2):
            p = f"blocks.{i}."
            mlp = {k_.replace(p + "ff.", "mlp."): v_ for k_, v_ in w32.items() if k_.startswith(p + "ff.")}
            h = P.rms_norm(x, w32[p + "n1.weight"], 1e-5)
            q = P.rope_neox(P.linear(h, w32[p + "attn.q_proj.weight"]).view(T, 2, 16), pos, 1e4)
            k = P.rope_neox(P.linear(h, w32[p + "attn.k_proj.weight"]).view(T, 2, 16), pos, 1e4)
            v = P.linear(h, w32[p + "attn.v_proj.weight"]).view(T, 2, 16)
            a = P.linear(P.causal_attention(q, k, v).reshape(T, 32), w32[p + "attn.o_proj.weight"])
            if i == 0:
                x = x + a + P.mlp_part(mlp, "", h)
            else:
                x = x + a
                x = x + P.mlp_part(mlp, "", P.rms_norm(x, w32[p + "n2.weight"], 1e-5))
        return P.linear(P.rms_norm(x, w32["final.weight"], 1e-5), w32["embed.weight"])
    e = Engine.from_tensors(cfg, w, dtype=dtype, max_tokens=256, max_slots=1)
    toks = random_tokens(30, 70, 8)
    s = e.alloc_slot()
    rows = [e.step([StepEntry(s, toks[:20], list(range(20)))])] + [e.step([StepEntry(s, [t], [0])]) for t in toks[20:]]
    e.free_slot(s)
    assert rel_l2(torch.cat(rows).cpu(), plain(toks)) < TOL[dtype]


# --------------------------------------------------------------------------- #
# A third kind of cache, an arrangement with four norms (and one layer without a feed-forward), an embedding
# multiplier and a logit scale, a checkpoint with fused q|k|v and gate|up tensors under other names, and a
# position encoding with an offset and a factor: all described by specs and registered here.
# --------------------------------------------------------------------------- #
def latent_parts():
    from titan_b200.cache import CacheGroup, CacheNeed, register_cache_group
    from titan_b200.cache.slots import CacheError
    from titan_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Mixer, Part, PositionEncoding
    from titan_b200.weights import WeightSpec

    class LatentGroup(CacheGroup):
        """One vector of ``width`` numbers per token and layer (no heads, no pages): [layers, slots, context, width]."""

        def __init__(self, need, layers, geometry):
            self.need, self.layers = need, list(layers)
            self.limit = geometry.max_context
            self.storage = torch.zeros((len(layers), geometry.max_slots, geometry.max_context, need.option("width")), device=geometry.device)
            self.held = {}

        def room_error(self, wanted):
            over = [s for s, n in wanted.items() if n > self.limit]
            return f"slots {over} would hold more than {self.limit} latent rows" if over else None

        def extend(self, slot, new_length):
            self.held[slot] = max(self.held.get(slot, 0), new_length)

        def release(self, slot, mark=False):
            if self.held.pop(slot, None) is not None and mark:
                self.storage[:, slot] = 3.0e4

        def check(self, is_live):
            for slot in self.held:
                if not is_live(slot):
                    raise CacheError(f"latent rows are held by slot {slot}, which is not live")

        def layer_storage(self, index_in_group):
            return self.storage[index_in_group]

        def bytes(self):
            return self.storage.numel() * 4
    register_cache_group("toy_latent", LatentGroup)

    class CausalMean(Mixer):
        """c_t = x_t . Wc^T is kept for every token; output_t = mean_{s <= t} c_s . Wo^T."""

        def __init__(self, spec):
            self.spec, self.width = spec, spec.option("latent", 8)

        def cache_need(self):
            return CacheNeed("toy_latent", extra=(("width", self.width),))

        def weight_specs(self, prefix):
            p = prefix + self.spec.prefix
            return [WeightSpec(p + "down.weight", (self.width, self.spec.hidden_size)), WeightSpec(p + "up.weight", (self.spec.hidden_size, self.width))]

        def bind(self, get):
            self.wc, self.wo = get(self.spec.prefix + "down.weight"), get(self.spec.prefix + "up.weight")

        def forward(self, h, ctx, cache, out):
            group, index = cache
            rows = group.layer_storage(index)                       # [slots, context, width]
            lay = ctx.layout
            c = (h.float() @ self.wc.float().t())
            starts, slots, first = lay.q_start.tolist(), lay.slot_of_seq.tolist(), lay.start_pos.tolist()
            for b, slot in enumerate(slots):
                n = starts[b + 1] - starts[b]
                rows[slot, first[b]:first[b] + n] = c[starts[b]:starts[b + 1]]
                sums = rows[slot, :first[b] + n].cumsum(0)[first[b]:]
                mean = sums / torch.arange(first[b] + 1, first[b] + n + 1, device=h.device)[:, None]
                out[starts[b]:starts[b + 1]] += mean.to(h.dtype).float() @ self.wo.float().t()
    MIXERS.register("toy_causal_mean", CausalMean)

    class Sandwich(Part):
        """x += norm_b(mixer(norm_a(x))); x += norm_d(feed_forward(norm_c(x))): a norm after each part as well as
        before it (the two after come from ``LayerSpec.norms``); a layer may have no feed-forward at all."""

        def __init__(self, spec):
            self.spec = spec
            self.pre_mixer, self.mixer = NORMS.build(spec.mixer_norm), MIXERS.build(spec.mixer)
            self.post_mixer = NORMS.build(spec.norms[0])
            self.has_ff = spec.feed_forward is not None
            if self.has_ff:
                self.pre_ff, self.feed_forward = NORMS.build(spec.feed_forward_norm), FEED_FORWARDS.build(spec.feed_forward)
                self.post_ff = NORMS.build(spec.norms[1])

        def parts(self):
            return (self.pre_mixer, self.mixer, self.post_mixer) + ((self.pre_ff, self.feed_forward, self.post_ff) if self.has_ff else ())

        def weight_specs(self, prefix=""):
            return [w for part in self.parts() for w in part.weight_specs(self.spec.prefix)]

        def bind(self, get):
            for part in self.parts():
                part.bind(lambda name: get(self.spec.prefix + name))

        def forward(self, x, ctx, cache):
            y = torch.zeros_like(x)
            self.mixer.forward(self.pre_mixer.forward(x, ctx), ctx, cache, y)
            x += self.post_mixer.forward(y, ctx).float()
            if self.has_ff:
                y = torch.zeros_like(x)
                self.feed_forward.forward(self.pre_ff.forward(x, ctx), ctx, y)
                x += self.post_ff.forward(y, ctx).float()
    BLOCKS.register("toy_sandwich", Sandwich)

    class ShiftedRotary(PositionEncoding):
        """Rotary angles of (position + shift), cosines and sines scaled by ``factor``: the mixer hands the block
        to its kernels as it is."""

        def __init__(self, spec):
            self.spec = spec
            self._inv = None

        @property
        def rotary_dim(self):
            return self.spec.rotary_dim

        def kernel_args(self, device):
            from titan_b200 import kernels as K
            if self._inv is None:
                k = torch.arange(self.spec.rotary_dim // 2, dtype=torch.float64)
                self._inv = (torch.tensor(self.spec.theta, dtype=torch.float64) ** (-2.0 * k / self.spec.rotary_dim)).float().to(device)
            return K.RotaryArgs(self._inv.data_ptr(), self.spec.rotary_dim, 3.0, 1.25)
    POSITIONS.register("toy_shifted_rope", ShiftedRotary)


class LatentConfig:
    def __init__(self, d):
        self.d = d

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def to_dict(self):
        return dict(self.d)

    def to_model_spec(self):
        from titan_b200.config import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
        d, H = self.d, self.d["width"]
        norm = lambda name: NormSpec("rmsnorm", H, 1e-5, name)
        layers = []
        for i in range(3):
            if i == 1:
                mixer = MixerSpec("attention", H, 4, 2, 16, position=PositionSpec("toy_shifted_rope", 16, 100.0), prefix="att.",
                                  names=(("qkv", "wqkv.weight"), ("o", "wo.weight")))
            else:
                mixer = MixerSpec("toy_causal_mean", H, prefix="mean.", extra=(("latent", d["latent"]),))
            ff = None if i == 2 else FeedForwardSpec("gated_mlp", H, d["ff"], prefix="ff.", names=(("gate_up", "w13.weight"), ("down", "w2.weight")))
            layers.append(LayerSpec(i, "toy_sandwich", mixer, ff, norm("a.weight"), None if ff is None else norm("c.weight"), f"blocks.{i}.",
                                    norms=(norm("b.weight"),) if ff is None else (norm("b.weight"), norm("d.weight"))))
        return ModelSpec("LatentForCausalLM", H, d["vocab"], tuple(layers), (0, 1, 2), norm("final.weight"), embedding="embed.weight",
                         lm_head=None, embedding_scale=d["embedding_scale"], logit_scale=d["logit_scale"])


def latent_plain(d, w, tokens):
    H, T = d["width"], len(tokens)
    x = w["embed.weight"][torch.tensor(tokens)] * d["embedding_scale"]
    pos = torch.arange(T)
    for i in range(3):
        p = f"blocks.{i}."
        h = P.rms_norm(x, w[p + "a.weight"], 1e-5)
        if i == 1:
            qkv = P.linear(h, w[p + "att.wqkv.weight"])
            q, k, v = qkv[:, :64].view(T, 4, 16), qkv[:, 64:96].view(T, 2, 16), qkv[:, 96:].view(T, 2, 16)
            q, k = 1.25 * P.rope_neox(q, pos + 3, 100.0), 1.25 * P.rope_neox(k, pos + 3, 100.0)
            y = P.linear(P.causal_attention(q, k, v).reshape(T, 64), w[p + "att.wo.weight"])
        else:
            c = P.linear(h, w[p + "mean.down.weight"])
            y = P.linear(c.cumsum(0) / torch.arange(1, T + 1)[:, None], w[p + "mean.up.weight"])
        x = x + P.rms_norm(y, w[p + "b.weight"], 1e-5)
        if i != 2:
            h = P.rms_norm(x, w[p + "c.weight"], 1e-5)
            both = w[p + "ff.w13.weight"]
            F = both.shape[0] // 2
            y = P.linear(P.swiglu(P.linear(h, both[:F]), P.linear(h, both[F:])), w[p + "ff.w2.weight"])
            x = x + P.rms_norm(y, w[p + "d.weight"], 1e-5)
    return P.linear(P.rms_norm(x, w["final.weight"], 1e-5), w["embed.weight"]) * d["logit_scale"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_third_cache_kind_four_norms_scales_and_other_tensor_names(dtype):
    from titan_b200 import Engine, StepEntry, StepError, register_architecture
    from titan_b200.parts import declare_weights
    latent_parts()
    register_architecture("LatentForCausalLM", LatentConfig)
    d = {"architectures": ["LatentForCausalLM"], "width": 64, "latent": 24, "ff": 96, "vocab": 130, "embedding_scale": 8.0, "logit_scale": 0.25}
    cfg = LatentConfig(d)
    g = torch.Generator().manual_seed(14)
    w = {}
    for s in declare_weights(cfg.to_model_spec()):
        t = torch.randn(s.shape, generator=g) * (0.1 if s.role == "vector" else 0.12) + (1.0 if s.role == "vector" else 0.0)
        w[s.name] = t.to(torch.bfloat16)
    assert "blocks.1.att.wqkv.weight" in w and "blocks.0.ff.w13.weight" in w and not any("q_proj" in n or "gate_proj" in n for n in w)
    assert not any(n.startswith("blocks.2.ff") or n.startswith("blocks.2.c.") for n in w)              # the last layer has no feed-forward
    e = Engine.from_tensors(cfg, w, dtype=dtype, max_tokens=256, max_context=128, max_slots=2, mark_freed_pages=True)
    assert sorted(type(g_).__name__ for g_ in e.cache.groups) == ["KVGroup", "LatentGroup"]
    w32 = {k: v.float() for k, v in w.items()}
    reqs = [random_tokens(90, 130, 1), random_tokens(33, 130, 2)]
    want = [latent_plain(d, w32, r) for r in reqs]
    for round_ in range(2):                                                  # slots, pages and latent rows are used again
        slots = [e.alloc_slot(), e.alloc_slot()]
        cut = [50, 4]
        out = e.step([StepEntry(slots[i], reqs[i][:cut[i]], list(range(cut[i]))) for i in range(2)])
        got, at = [[out[:cut[0]]], [out[cut[0]:]]], list(cut)
        out = e.step([StepEntry(slots[0], reqs[0][50:70], list(range(20)))])  # a continuation chunk
        got[0].append(out)
        at[0] = 70
        while any(a < len(r) for a, r in zip(at, reqs)):
            live = [i for i in range(2) if at[i] < len(reqs[i])]
            out = e.step([StepEntry(slots[i], [reqs[i][at[i]]], [0]) for i in live])
            for k, i in enumerate(live):
                got[i].append(out[k:k + 1])
                at[i] += 1
        for i in range(2):
            assert rel_l2(torch.cat(got[i]).cpu(), want[i]) < TOL[dtype], (round_, i)
        with pytest.raises(StepError, match="context"):
            e.step([StepEntry(slots[0], [1] * 39, [])])                        # 90 + 39 > 128
        e.cache.check()
        for s in slots:
            e.free_slot(s)
    e.cache.check()
    assert [g_.held for g_ in e.cache.groups if type(g_).__name__ == "LatentGroup"] == [{}]
