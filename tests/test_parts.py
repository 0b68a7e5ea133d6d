"""The parts of a layer alone, the run order as data, and a toy mixer with state
of its own that is registered, built and stepped without touching the library's
files.  Every test runs on the GPU (``-m gpu``); the same bodies also run on the
CPU with the kernels swapped for their plain restatements, which checks the
Python side (wiring, cache, batching) where there is no GPU."""

import math

import pytest
import torch

import simple_inference_autoresearch_b200 as siar
from simple_inference_autoresearch_b200 import StepEntry, registry
from simple_inference_autoresearch_b200.config import LlamaConfig
from simple_inference_autoresearch_b200.engine.batch import BatchMeta
from simple_inference_autoresearch_b200.engine.model import DecoderModel, ModelSpec, ScheduleEntry, StepContext
from simple_inference_autoresearch_b200.architectures.llama import llama_model_spec
from simple_inference_autoresearch_b200.cache import SequenceCache
from simple_inference_autoresearch_b200.parts import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS,
                                                      Block, FeedForward, Mixer, Norm, PartSpec, PositionEncoding,
                                                      StateNeed, TensorSpec)
from simple_inference_autoresearch_b200.weights import random_tensors
from tests import emulated_kernels, plain_llama, tiny_configs

DEVICES = [pytest.param("cpu", id="cpu-emulated"), pytest.param("cuda", marks=pytest.mark.gpu, id="gpu")]


@pytest.fixture(params=DEVICES)
def device(request, monkeypatch):
    if request.param == "cpu":
        emulated_kernels.install(monkeypatch)
    return request.param


def tensors_for(part, seed, dtype, device):
    return {k: v.to(device) for k, v in random_tensors(part.tensor_specs(), seed, dtype).items()}


def meta_for(device, q_lens, base_lens, slots):
    return BatchMeta.build([StepEntry(s, [0] * n) for s, n in zip(slots, q_lens)], base_lens, device)


# ----------------------------------------------------------------------------- parts alone
def test_norm_part(device):
    norm = NORMS.build(PartSpec("rmsnorm", {"prefix": "n.", "hidden_size": 80, "eps": 1e-6,
                                            "weight_init": "ones_plus_normal"}))
    assert [s.name for s in norm.tensor_specs()] == ["n.weight"]
    w = tensors_for(norm, 1, torch.float32, device)
    norm.load(w)
    ctx = StepContext(torch.float32, None, None)
    res = torch.randn(5, 80, generator=torch.Generator().manual_seed(0))
    delta = torch.randn(5, 80, generator=torch.Generator().manual_seed(1))
    r = res.clone().to(device)
    out = norm.add_norm(ctx, r, delta.to(device))
    torch.testing.assert_close(r.cpu(), res + delta)
    torch.testing.assert_close(out.cpu(), plain_llama.rmsnorm(res + delta, w["n.weight"].cpu(), 1e-6),
                               rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(norm.norm(ctx, r).cpu(), out.cpu())


def test_position_part_matches_the_reference_frequencies():
    for raw in (tiny_configs.TINY_A, tiny_configs.TINY_B):
        d = raw.get("head_dim") or raw["hidden_size"] // raw["num_attention_heads"]
        pos = POSITION_ENCODINGS.build(PartSpec("rotary", {"head_dim": d, "theta": raw["rope_theta"],
                                                           "scaling": raw["rope_scaling"]}))
        want = plain_llama.rope_inv_freq(d, raw["rope_theta"], raw["rope_scaling"])
        assert torch.equal(pos.rotary().inv_freq, want)
    assert POSITION_ENCODINGS.build(PartSpec("none")).rotary() is None


def test_feed_forward_part(device):
    ffn = FEED_FORWARDS.build(PartSpec("swiglu", {"prefix": "m.", "hidden_size": 80, "intermediate_size": 136}))
    w = tensors_for(ffn, 2, torch.float32, device)
    ffn.load(w)
    x = torch.randn(7, 80, generator=torch.Generator().manual_seed(3))
    out = ffn.forward(StepContext(torch.float32, None, None), x.to(device))
    ref = plain_llama.swiglu_mlp(x, {k: v.cpu() for k, v in w.items()}, "m.")
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-5, atol=1e-6)


def test_mixer_part_over_a_cache(device):
    """The attention mixer alone: a prompt in one step, then two single tokens,
    equals the plain attention block over the whole sequence."""
    c = {"H": 80, "Hq": 6, "Hkv": 2, "D": 48}
    pos = POSITION_ENCODINGS.build(PartSpec("rotary", {"head_dim": 48, "theta": 10000.0, "scaling": None}),
                                   device=device)
    mixer = MIXERS.build(PartSpec("gqa_attention", {"prefix": "a.", "hidden_size": 80, "n_heads": 6,
                                                    "n_kv_heads": 2, "head_dim": 48}), position=pos)
    w = tensors_for(mixer, 4, torch.float32, device)
    mixer.load(w)
    cache = SequenceCache([mixer.cache_need()], 256, 2, 128, torch.float32, device)
    decoy, s = cache.alloc(), cache.alloc()
    x = torch.randn(12, 80, generator=torch.Generator().manual_seed(5))
    outs, done = [], 0
    for n in (10, 1, 1):
        cache.reserve([s], [n])
        ctx = StepContext(torch.float32, meta_for(device, [n], [done], [s]), cache)
        outs.append(mixer.forward(ctx, x[done:done + n].contiguous().to(device), cache.entry(0), True).cpu())
        cache.commit([s], [n])
        done += n
    ref = plain_llama.attention_block(x, {k: v.cpu() for k, v in w.items()}, "a.", c,
                                      plain_llama.rope_inv_freq(48, 10000.0, None))
    torch.testing.assert_close(torch.cat(outs), ref, rtol=2e-5, atol=2e-6)


def test_block_part_threads_the_residual(device):
    cfg = LlamaConfig.from_dict(tiny_configs.TINY_C)
    spec = llama_model_spec(cfg, norm_weight_init="ones_plus_normal")
    pos = POSITION_ENCODINGS.build(spec.position, device=device)
    blk = BLOCKS.build(spec.layers[1], position=pos)
    w = tensors_for(blk, 6, torch.float32, device)
    blk.load(w)
    cache = SequenceCache([blk.cache_need()], 128, 1, 64, torch.float32, device)
    s = cache.alloc()
    cache.reserve([s], [9])
    ctx = StepContext(torch.float32, meta_for(device, [9], [0], [s]), cache)
    x = torch.randn(9, 80, generator=torch.Generator().manual_seed(7))
    pending = torch.randn(9, 80, generator=torch.Generator().manual_seed(8))
    residual, m = blk.forward(ctx, x.clone().to(device), pending.to(device), cache.entry(0), True)
    c = plain_llama.parse_config(tiny_configs.TINY_C)
    ref = plain_llama.block(x + pending, {k: v.cpu() for k, v in w.items()}, 1, c,
                            plain_llama.rope_inv_freq(c["D"], c["theta"], None))
    torch.testing.assert_close((residual + m).cpu(), ref, rtol=2e-5, atol=2e-6)


# ----------------------------------------------------------------------------- the run order is data
def test_schedule_may_repeat_a_layer_and_share_a_cache(device, tmp_path):
    """Layer 0 runs twice (two cache entries of its own), and the last run reads
    the cache that the run of layer 1 wrote instead of writing one."""
    folder = tiny_configs.make_folder(tmp_path, "C", seed=3)
    raw, w = tiny_configs.read_folder(folder)
    cfg = LlamaConfig.from_dict(raw)
    base = llama_model_spec(cfg)
    sched = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(1, 1, writes_cache=False))
    spec = ModelSpec(**{**base.__dict__, "schedule": sched})
    model = DecoderModel(spec, torch.float32, device)
    assert len(model.cache_needs) == 3
    model.load({k: v.float().to(device) for k, v in w.items()})
    eng = siar.Engine(model, max_batch=2, max_seq_len=128, use_cuda_graph=False)
    toks = torch.randint(0, raw["vocab_size"], (45,), generator=torch.Generator().manual_seed(2)).tolist()
    s = eng.open()
    outs = [eng.step([StepEntry(s, toks[:30], range(30))])]
    outs += [eng.step([StepEntry(s, [t], [0])]) for t in toks[30:]]
    ref = plain_llama.forward(w, raw, toks, schedule=[(e.layer, e.cache_entry, e.writes_cache) for e in sched])
    torch.testing.assert_close(torch.cat(outs).cpu(), ref, rtol=2e-5, atol=2e-5)
    plain = plain_llama.forward(w, raw, toks)
    assert (ref - plain).abs().max() > 1e-3     # the schedule really changes the function
    for bad in ((ScheduleEntry(0, 0), ScheduleEntry(1, 0)),                        # two writers of one entry
                (ScheduleEntry(0, 1, writes_cache=False), ScheduleEntry(1, 1)),     # read before write
                (ScheduleEntry(5, 0),)):                                            # no such layer
        with pytest.raises(ValueError):
            DecoderModel(ModelSpec(**{**base.__dict__, "schedule": bad}), torch.float32, device)


def test_layers_with_a_window_get_a_cache_group_of_their_own(device, tmp_path):
    """Layer 0 keeps all keys, layers 1 and 2 the last 37 (no multiple of a page, shorter than the
    prompt): two storage groups; whole prompt, then one token at a time far past the window,
    against the plain implementation with the same masks; the windowed group holds a bounded
    number of pages meanwhile and every page is free at the end."""
    folder = tiny_configs.make_folder(tmp_path, "B", seed=5)        # three layers
    raw, w = tiny_configs.read_folder(folder)
    cfg = LlamaConfig.from_dict(raw)
    base = llama_model_spec(cfg)
    window = 37
    layers = list(base.layers)
    for i in (1, 2):
        p = dict(layers[i].params)
        p["mixer"] = PartSpec("gqa_attention", {**p["mixer"].params, "window": window})
        layers[i] = PartSpec(layers[i].kind, p)
    model = DecoderModel(ModelSpec(**{**base.__dict__, "layers": tuple(layers)}), torch.float32, device)
    assert model.cache_needs[0].window is None and model.cache_needs[1].window == window
    model.load({k: v.float().to(device) for k, v in w.items()})
    eng = siar.Engine(model, max_batch=2, max_seq_len=256, use_cuda_graph=False)
    full, win = eng.cache.groups
    assert full.need.window is None and win.need.window == window and win.n_entries == 2
    g = torch.Generator().manual_seed(4)
    toks = torch.randint(0, raw["vocab_size"], (150,), generator=g).tolist()
    other = torch.randint(0, raw["vocab_size"], (20,), generator=g).tolist()
    a, b = eng.open(), eng.open()
    outs = [eng.step([StepEntry(a, toks[:90], range(90)), StepEntry(b, other, [])])[:90]]
    for t in toks[90:]:
        outs.append(eng.step([StepEntry(a, [t], [0])]))
        assert win.held_pages(a) <= 2 and full.held_pages(a) == -(-eng.cache.length(a) // 64)
    ref = plain_llama.forward(w, raw, toks, windows={1: window, 2: window})
    torch.testing.assert_close(torch.cat(outs).cpu(), ref, rtol=2e-5, atol=2e-5)
    assert (ref - plain_llama.forward(w, raw, toks)).abs().max() > 1e-3      # the window really matters
    eng.close(a); eng.close(b)
    assert len(win.pages) == win.pages.n and len(full.pages) == full.pages.n


# ----------------------------------------------------------------------------- a toy mixer with state of its own
class RunningMeanMixer(Mixer):
    """y_t = W * mean(x_0 .. x_t): per-sequence state = (sum [H], count [1]).
    Written with torch ops; it stands for a mixer that is not attention."""

    def __init__(self, prefix, position, hidden_size):
        super().__init__(prefix)
        self.h = hidden_size
        self.w = None

    def tensor_specs(self):
        return [TensorSpec(self.prefix + "w", (self.h, self.h), std=0.1)]

    def load(self, tensors):
        self.w = tensors[self.prefix + "w"]

    def cache_need(self):
        return StateNeed((self.h + 1,), "float32")

    def forward(self, ctx, x, cache_entry, writes_cache=True):
        m, st = ctx.meta, cache_entry.state
        out = torch.empty(x.shape[0], self.h, dtype=torch.float32, device=x.device)
        row = 0
        for slot, n in zip(m.slots, m.q_lens):
            xs = x[row:row + n].float()
            sums = st[slot, :self.h] + torch.cumsum(xs, 0)
            counts = st[slot, self.h] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
            out[row:row + n] = (sums / counts[:, None]) @ self.w.float().T
            st[slot, :self.h] = sums[-1]
            st[slot, self.h] = counts[-1]
            row += n
        return out


def toy_spec(cfg_like, **_):
    h, v = cfg_like.hidden_size, cfg_like.vocab_size
    norm = lambda p: PartSpec("rmsnorm", {"prefix": p, "hidden_size": h, "eps": 1e-5})  # noqa: E731
    attn = PartSpec("gqa_attention", {"prefix": "attn.", "hidden_size": h, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16})
    toy = PartSpec("running_mean", {"prefix": "mix.", "hidden_size": h})
    ffn = PartSpec("swiglu", {"prefix": "ffn.", "hidden_size": h, "intermediate_size": 40})
    layer = lambda i, mixer: PartSpec("prenorm", {"prefix": f"l{i}.", "mixer": mixer, "feed_forward": ffn,  # noqa: E731
                                                  "mixer_norm": norm("n1."), "ffn_norm": norm("n2.")})
    return ModelSpec(architecture="ToyForCausalLM", vocab_size=v, hidden_size=h, max_position=128,
                     embedding_name="emb", head_name=None,
                     position=PartSpec("rotary", {"head_dim": 16, "theta": 10000.0, "scaling": None}),
                     layers=(layer(0, toy), layer(1, attn), layer(2, toy)), final_norm=norm("nf."))


def toy_plain(w, h, tokens):
    """The toy model written out plainly, whole sequence, for comparison."""
    x = w["emb"][torch.tensor(tokens)]
    c = {"H": h, "Hq": 2, "Hkv": 1, "D": 16}
    inv = plain_llama.rope_inv_freq(16, 10000.0, None)
    for i in range(3):
        p = f"l{i}."
        hn = plain_llama.rmsnorm(x, w[p + "n1.weight"], 1e-5)
        if i == 1:
            a = plain_llama.attention_block(hn, w, p + "attn.", c, inv)
        else:
            mean = torch.cumsum(hn, 0) / torch.arange(1, len(tokens) + 1)[:, None]
            a = mean @ w[p + "mix.w"].T
        x = x + a
        x = x + plain_llama.swiglu_mlp(plain_llama.rmsnorm(x, w[p + "n2.weight"], 1e-5), w, p + "ffn.")
    return plain_llama.rmsnorm(x, w["nf.weight"], 1e-5) @ w["emb"].T


def test_toy_mixer_with_its_own_state_registers_builds_and_steps(device):
    MIXERS.register("running_mean")(RunningMeanMixer)
    registry.register_architecture("ToyForCausalLM", ("toy",), config_cls=LlamaConfig, spec_builder=toy_spec)
    try:
        class Cfg:
            hidden_size, vocab_size = 32, 50
        arch = registry.resolve({"architectures": ["ToyForCausalLM"]})
        model = DecoderModel(arch.spec_builder(Cfg), torch.float32, device)
        kinds = [type(n).__name__ for n in model.cache_needs]
        assert kinds == ["StateNeed", "KVNeed", "StateNeed"]
        w = random_tensors(model.tensor_specs(), 9, torch.float32)
        model.load({k: v.to(device) for k, v in w.items()})
        eng = siar.Engine(model, max_batch=3, max_seq_len=128, use_cuda_graph=False)
        g = torch.Generator().manual_seed(4)
        reqs = [torch.randint(0, 50, (n,), generator=g).tolist() for n in (20, 7, 33)]
        for rounds in range(2):                 # second round reuses the slots: state must start from zero
            slots = [eng.open() for _ in reqs]
            got = [[] for _ in reqs]
            heads = [len(r) - 5 for r in reqs]
            out = eng.step([StepEntry(s, r[:h], range(h)) for s, r, h in zip(slots, reqs, heads)])
            o = 0
            for i, h in enumerate(heads):
                got[i].append(out[o:o + h]); o += h
            for k in range(5):
                out = eng.step([StepEntry(s, [r[h + k]], [0]) for s, r, h in zip(slots, reqs, heads)])
                for i in range(len(reqs)):
                    got[i].append(out[i:i + 1])
            for i, r in enumerate(reqs):
                torch.testing.assert_close(torch.cat(got[i]).cpu(), toy_plain(w, 32, r), rtol=2e-5, atol=2e-5)
            for s in slots:
                eng.close(s)
    finally:
        MIXERS.unregister("running_mean")
        registry.unregister_architecture("ToyForCausalLM")


# ----------------------------------------------------------------------------- a toy feed-forward with routing,
# ----------------------------------------------------------------------------- a toy position encoding that adds at the embedding
class RoutedFeedForward(FeedForward):
    """Top-1 routing over E small experts, y = gate_prob * (relu(x W1_e) W2_e); router logits and
    the softmax in 32-bit.  Torch ops; it stands for a feed-forward that is not dense."""

    def __init__(self, prefix, hidden_size, n_experts, expert_size):
        super().__init__(prefix)
        self.h, self.e, self.f = hidden_size, n_experts, expert_size
        self.router = self.w1 = self.w2 = None

    def tensor_specs(self):
        p = self.prefix
        return [TensorSpec(p + "router", (self.e, self.h), std=0.5),
                TensorSpec(p + "w1", (self.e, self.f, self.h), std=0.1),
                TensorSpec(p + "w2", (self.e, self.h, self.f), std=0.1)]

    def load(self, tensors):
        p = self.prefix
        self.router, self.w1, self.w2 = tensors[p + "router"], tensors[p + "w1"], tensors[p + "w2"]

    def forward(self, ctx, x):
        return routed_ffn_plain(x.float(), self.router.float(), self.w1.float(), self.w2.float())


def routed_ffn_plain(x, router, w1, w2):
    probs = torch.softmax(x @ router.T, dim=-1)
    top = probs.argmax(dim=-1)
    out = torch.zeros_like(x)
    for e in range(router.shape[0]):
        rows = (top == e).nonzero().flatten()
        if rows.numel():
            out[rows] = probs[rows, e:e + 1] * (torch.relu(x[rows] @ w1[e].T) @ w2[e].T)
    return out


class LearnedPositions(PositionEncoding):
    """Absolute positions: a learned table row is added to each embedded token; mixers get no rotation."""

    def __init__(self, prefix="pos.", *, hidden_size, max_position, device=None):
        super().__init__(prefix)
        self.h, self.n = hidden_size, max_position
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.prefix + "table", (self.n, self.h), std=0.1)]

    def load(self, tensors):
        self.table = tensors[self.prefix + "table"]

    def at_embedding(self, ctx, residual):
        m = ctx.meta
        pos = torch.cat([torch.arange(b, b + n) for b, n in zip(m.base_lens, m.q_lens)]).to(residual.device)
        residual += self.table[pos].float()


def test_toy_routed_feed_forward_and_learned_positions(device):
    """Two more parts from outside the library: a routed feed-forward and a position encoding that
    enters at the embedding, in a model whose layers differ (layer 0 dense, layer 1 routed)."""
    FEED_FORWARDS.register("routed")(RoutedFeedForward)
    POSITION_ENCODINGS.register("learned")(LearnedPositions)
    try:
        h, v = 32, 40
        norm = lambda p: PartSpec("rmsnorm", {"prefix": p, "hidden_size": h, "eps": 1e-5})  # noqa: E731
        attn = PartSpec("gqa_attention", {"prefix": "attn.", "hidden_size": h, "n_heads": 2, "n_kv_heads": 2, "head_dim": 16})
        dense = PartSpec("swiglu", {"prefix": "ffn.", "hidden_size": h, "intermediate_size": 48})
        routed = PartSpec("routed", {"prefix": "moe.", "hidden_size": h, "n_experts": 3, "expert_size": 24})
        layer = lambda i, ffn: PartSpec("prenorm", {"prefix": f"l{i}.", "mixer": attn, "feed_forward": ffn,  # noqa: E731
                                                    "mixer_norm": norm("n1."), "ffn_norm": norm("n2.")})
        spec = ModelSpec(architecture="Toy2", vocab_size=v, hidden_size=h, max_position=64, embedding_name="emb",
                         head_name="head", position=PartSpec("learned", {"hidden_size": h, "max_position": 64}),
                         layers=(layer(0, dense), layer(1, routed)), final_norm=norm("nf."))
        model = DecoderModel(spec, torch.float32, device)
        assert "pos.table" in [t.name for t in model.tensor_specs()]
        w = random_tensors(model.tensor_specs(), 5, torch.float32)
        model.load({k: t.to(device) for k, t in w.items()})
        eng = siar.Engine(model, max_batch=2, max_seq_len=64, use_cuda_graph=False)
        g = torch.Generator().manual_seed(6)
        reqs = [torch.randint(0, v, (n,), generator=g).tolist() for n in (19, 8)]
        slots = [eng.open() for _ in reqs]
        got = [[] for _ in reqs]
        out = eng.step([StepEntry(s, r[:-3], range(len(r) - 3)) for s, r in zip(slots, reqs)])
        o = 0
        for i, r in enumerate(reqs):
            got[i].append(out[o:o + len(r) - 3]); o += len(r) - 3
        for k in range(3):
            out = eng.step([StepEntry(s, [r[len(r) - 3 + k]], [0]) for s, r in zip(slots, reqs)])
            for i in range(len(reqs)):
                got[i].append(out[i:i + 1])
        for i, r in enumerate(reqs):          # the same model written out plainly, whole sequence
            x = w["emb"][torch.tensor(r)] + w["pos.table"][:len(r)]
            c = {"H": h, "Hq": 2, "Hkv": 2, "D": 16}
            for li, ffn in ((0, "dense"), (1, "routed")):
                p = f"l{li}."
                hn = plain_llama.rmsnorm(x, w[p + "n1.weight"], 1e-5)
                t = len(r)
                q = (hn @ w[p + "attn.q_proj.weight"].T).view(t, 2, 16)       # no rotation in this model
                kk = (hn @ w[p + "attn.k_proj.weight"].T).view(t, 2, 16)
                vv = (hn @ w[p + "attn.v_proj.weight"].T).view(t, 2, 16)
                x = x + plain_llama.attention_causal(q, kk, vv) @ w[p + "attn.o_proj.weight"].T
                hn = plain_llama.rmsnorm(x, w[p + "n2.weight"], 1e-5)
                if ffn == "dense":
                    x = x + plain_llama.swiglu_mlp(hn, w, p + "ffn.")
                else:
                    x = x + routed_ffn_plain(hn, w[p + "moe.router"], w[p + "moe.w1"], w[p + "moe.w2"])
            ref = plain_llama.rmsnorm(x, w["nf.weight"], 1e-5) @ w["head"].T
            torch.testing.assert_close(torch.cat(got[i]).cpu(), ref, rtol=2e-5, atol=2e-5)
    finally:
        FEED_FORWARDS.unregister("routed")
        POSITION_ENCODINGS.unregister("learned")


# ----------------------------------------------------------------------------- a toy norm and a toy arrangement of a block
class BiasedLayerNorm(Norm):
    """y = (x - mean(x)) * rsqrt(var(x) + eps) * w + b, all in 32-bit.  Torch ops; it stands for a norm
    the product kernels cannot take over (it gives no hint, so nothing is deferred to a product)."""

    def __init__(self, prefix, hidden_size, eps):
        super().__init__(prefix)
        self.h, self.eps = hidden_size, eps
        self.w = self.b = None

    def tensor_specs(self):
        return [TensorSpec(self.prefix + "w", (self.h,), role="vector", init="ones_plus_normal", std=0.1),
                TensorSpec(self.prefix + "b", (self.h,), role="vector", init="normal", std=0.1)]

    def load(self, tensors):
        self.w, self.b = tensors[self.prefix + "w"], tensors[self.prefix + "b"]

    def norm(self, ctx, residual):
        x = residual.float()
        x = x - x.mean(-1, keepdim=True)
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.w.float() + self.b.float()
        return y.to(ctx.dtype)

    def add_norm(self, ctx, residual, delta):
        residual.add_(delta.float())
        return self.norm(ctx, residual)


class ParallelBlock(Block):
    """x += mixer(norm(x)) + ffn(norm(x)): one norm, both sublayers read the same normed input."""

    def __init__(self, prefix, position, mixer, feed_forward, norm):
        super().__init__(prefix)
        at = lambda spec: PartSpec(spec.kind, {**spec.params, "prefix": prefix + spec.params.get("prefix", "")})  # noqa: E731
        self.norm_part = NORMS.build(at(norm))
        self.mixer = MIXERS.build(at(mixer), position=position)
        self.ffn = FEED_FORWARDS.build(at(feed_forward))
        self._parts = [self.norm_part, self.mixer, self.ffn]

    def tensor_specs(self):
        return [s for p in self._parts for s in p.tensor_specs()]

    def load(self, tensors):
        for p in self._parts:
            p.load(tensors)

    def extension_units(self, dtype=None):
        units = ()
        for p in self._parts:
            units += tuple(p.extension_units(dtype))
        return units

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, ctx, residual, pending, cache_entry, writes_cache=True):
        from simple_inference_autoresearch_b200.kernels import ops
        ctx.residual, ctx.next_norm = residual, None
        if pending is None or isinstance(pending, ops.Added):       # nothing to add, or already added by its product
            h = self.norm_part.norm(ctx, residual)
        else:
            h = self.norm_part.add_norm(ctx, residual, pending)
        for out in (self.mixer.forward(ctx, h, cache_entry, writes_cache), self.ffn.forward(ctx, h)):
            if not isinstance(out, ops.Added):                       # a product that did not add itself
                residual.add_(out.float())
        return residual, None


def parallel_spec(cfg_like, **_):
    h, v, d = cfg_like.hidden_size, cfg_like.vocab_size, cfg_like.head_dim
    ln = lambda p: PartSpec("layernorm_bias", {"prefix": p, "hidden_size": h, "eps": 1e-3})  # noqa: E731
    attn = PartSpec("gqa_attention", {"prefix": "attn.", "hidden_size": h, "n_heads": 2, "n_kv_heads": 1, "head_dim": d})
    ffn = PartSpec("swiglu", {"prefix": "ffn.", "hidden_size": h, "intermediate_size": 3 * h // 2})
    par = lambda i: PartSpec("parallel", {"prefix": f"l{i}.", "mixer": attn, "feed_forward": ffn, "norm": ln("ln.")})  # noqa: E731
    pre = PartSpec("prenorm", {"prefix": "l1.", "mixer": attn, "feed_forward": ffn,
                               "mixer_norm": PartSpec("rmsnorm", {"prefix": "n1.", "hidden_size": h, "eps": 1e-5}),
                               "ffn_norm": ln("n2.")})
    return ModelSpec(architecture="ParallelForCausalLM", vocab_size=v, hidden_size=h, max_position=256,
                     embedding_name="emb", head_name=None,
                     position=PartSpec("rotary", {"head_dim": d, "theta": 10000.0, "scaling": None}),
                     layers=(par(0), pre, par(2)), final_norm=ln("nf."))


def parallel_plain(w, h, d, tokens):
    """The model of ``parallel_spec`` written out plainly, whole sequence."""
    w = {k: v.float() for k, v in w.items()}

    def ln(x, p):
        x = x - x.mean(-1, keepdim=True)
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-3) * w[p + "w"] + w[p + "b"]

    c = {"H": h, "Hq": 2, "Hkv": 1, "D": d}
    inv = plain_llama.rope_inv_freq(d, 10000.0, None)
    x = w["emb"][torch.tensor(tokens)]
    for i in (0, 1, 2):
        p = f"l{i}."
        if i == 1:
            x = x + plain_llama.attention_block(plain_llama.rmsnorm(x, w[p + "n1.weight"], 1e-5), w, p + "attn.", c, inv)
            x = x + plain_llama.swiglu_mlp(ln(x, p + "n2."), w, p + "ffn.")
        else:
            hn = ln(x, p + "ln.")
            x = x + plain_llama.attention_block(hn, w, p + "attn.", c, inv) + plain_llama.swiglu_mlp(hn, w, p + "ffn.")
    return ln(x, "nf.") @ w["emb"].T


@pytest.mark.parametrize("dtype,hidden,head_dim", [(torch.float32, 40, 16), (torch.bfloat16, 128, 64)])
def test_toy_norm_and_toy_block_arrangement_register_build_and_step(device, dtype, hidden, head_dim):
    """A norm the product kernels know nothing of and a block that arranges its parts another way,
    both defined here, beside the library's own block in the middle layer: the products that add
    themselves into the residual and leave a norm's inputs behind must fall back where the norm
    that follows is not theirs."""
    NORMS.register("layernorm_bias")(BiasedLayerNorm)
    BLOCKS.register("parallel")(ParallelBlock)
    registry.register_architecture("ParallelForCausalLM", ("parallel_toy",), config_cls=LlamaConfig, spec_builder=parallel_spec)
    try:
        class Cfg:
            hidden_size, vocab_size = hidden, 70
        Cfg.head_dim = head_dim
        arch = registry.resolve({"architectures": ["ParallelForCausalLM"]})
        model = DecoderModel(arch.spec_builder(Cfg), dtype, device)
        w = random_tensors(model.tensor_specs(), 11, torch.float32)
        w = {k: v.to(dtype).float() for k, v in w.items()}           # what the model holds, exactly
        model.load({k: (v if v.dim() == 1 else v.to(dtype)).to(device) for k, v in w.items()})
        eng = siar.Engine(model, max_batch=3, max_seq_len=256, use_cuda_graph=False)
        g = torch.Generator().manual_seed(6)
        reqs = [torch.randint(0, 70, (n,), generator=g).tolist() for n in (150, 9, 41)]
        tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=4e-2, atol=4e-2)
        for rounds in range(2):
            slots = [eng.open() for _ in reqs]
            heads = [len(r) - 4 for r in reqs]
            got = [[] for _ in reqs]
            out = eng.step([StepEntry(s, r[:h], range(h)) for s, r, h in zip(slots, reqs, heads)])
            o = 0
            for i, h in enumerate(heads):
                got[i].append(out[o:o + h]); o += h
            for k in range(4):
                out = eng.step([StepEntry(s, [r[h + k]], [0]) for s, r, h in zip(slots, reqs, heads)])
                for i in range(len(reqs)):
                    got[i].append(out[i:i + 1])
            for i, r in enumerate(reqs):
                torch.testing.assert_close(torch.cat(got[i]).cpu(), parallel_plain(w, hidden, head_dim, r), **tol)
            for s in slots:
                eng.close(s)
    finally:
        NORMS.unregister("layernorm_bias")
        BLOCKS.unregister("parallel")
        registry.unregister_architecture("ParallelForCausalLM")


# ----------------------------------------------------------------------------- rotary layouts that are not Llama's
def plain_forward_with_rotary_layout(w, raw, tokens, rotary_dim, interleaved):
    """plain_llama.forward with the rotation of q and k replaced by a partial and / or interleaved one."""
    c = plain_llama.parse_config(raw)
    w = {k: v.float() for k, v in w.items()}
    inv = plain_llama.rope_inv_freq(rotary_dim, c["theta"], c["scaling"])
    t = len(tokens)
    x = w["model.embed_tokens.weight"][torch.tensor(tokens)]
    for i in range(c["L"]):
        p = f"model.layers.{i}."
        hn = plain_llama.rmsnorm(x, w[p + "input_layernorm.weight"], c["eps"])
        q = (hn @ w[p + "self_attn.q_proj.weight"].T).view(t, c["Hq"], c["D"])
        k = (hn @ w[p + "self_attn.k_proj.weight"].T).view(t, c["Hkv"], c["D"])
        v = (hn @ w[p + "self_attn.v_proj.weight"].T).view(t, c["Hkv"], c["D"])
        q = emulated_kernels.rotate(q, list(range(t)), inv, rotary_dim, interleaved)
        k = emulated_kernels.rotate(k, list(range(t)), inv, rotary_dim, interleaved)
        x = x + plain_llama.attention_causal(q, k, v) @ w[p + "self_attn.o_proj.weight"].T
        x = x + plain_llama.swiglu_mlp(plain_llama.rmsnorm(x, w[p + "post_attention_layernorm.weight"], c["eps"]), w, p + "mlp.")
    head = w["model.embed_tokens.weight"] if c["tied"] else w["lm_head.weight"]
    return plain_llama.rmsnorm(x, w["model.norm.weight"], c["eps"]) @ head.T


@pytest.mark.parametrize("name,dtype,rotary_dim,interleaved", [
    ("C", torch.float32, 32, True),        # head_dim 48: two thirds of a head rotated, pairs (2i, 2i+1)
    ("C", torch.float32, 48, True),
    ("D", torch.bfloat16, 32, False),      # head_dim 64 on the tensor-core path: half a head rotated
    ("E", torch.bfloat16, 128, True),
])
def test_partial_and_interleaved_rotary_are_parameters_of_the_position_encoding(device, tmp_path, name, dtype,
                                                                                rotary_dim, interleaved):
    """The Llama parts with another rotary layout, given as parameters of the ``rotary`` position
    encoding: whole prompt, then single tokens (on the bfloat16 tensor-core path the decode step
    cannot take the kernel that rotates inside attention and goes the two-kernel way)."""
    if device == "cpu" and dtype != torch.float32:
        pytest.skip("the emulated kernels check the wiring once, in float32")
    folder = tiny_configs.make_folder(tmp_path, name, seed=3)
    raw, w = tiny_configs.read_folder(folder)
    base = llama_model_spec(LlamaConfig.from_dict(raw))
    position = PartSpec("rotary", {**base.position.params, "rotary_dim": rotary_dim, "interleaved": interleaved})
    model = DecoderModel(ModelSpec(**{**base.__dict__, "position": position}), dtype, device)
    model.load({k: v.to(dtype).to(device) for k, v in w.items()})
    eng = siar.Engine(model, max_batch=2, max_seq_len=256, use_cuda_graph=False)
    toks = torch.randint(0, raw["vocab_size"], (90,), generator=torch.Generator().manual_seed(2)).tolist()
    s = eng.open()
    outs = [eng.step([StepEntry(s, toks[:70], range(70))])]
    outs += [eng.step([StepEntry(s, [t], [0])]) for t in toks[70:]]
    got = torch.cat(outs).float().cpu()
    ref = plain_forward_with_rotary_layout(w, raw, toks, rotary_dim, interleaved)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (got - ref).abs().max().item() <= tol * ref.abs().max().item()
    assert (ref - plain_llama.forward(w, raw, toks)).abs().max() > 1e-3        # the layout really matters
    with pytest.raises(ValueError, match="rotary_dim"):
        POSITION_ENCODINGS.build(PartSpec("rotary", {"head_dim": 16, "theta": 1e4, "rotary_dim": 18}))


# ----------------------------------------------------------------------------- another architecture from outside, through the command line
class ToyConfig:
    """The typed configuration of an architecture that is not Llama: its own config.json keys."""

    def __init__(self, width, vocab, depth, stop):
        self.width, self.vocab, self.depth, self.stop = width, vocab, depth, stop
        self.vocab_size, self.bos_token_id = vocab, 0          # what the command line reads of any configuration

    @classmethod
    def from_dict(cls, d):
        return cls(int(d["width"]), int(d["vocab"]), int(d["depth"]), int(d.get("stop", 1)))

    def to_dict(self):
        return {"architectures": ["ToyMeanForCausalLM"], "model_type": "toy_mean", "width": self.width,
                "vocab": self.vocab, "depth": self.depth, "stop": self.stop}


def toy_mean_spec(cfg, **_):
    norm = lambda p: PartSpec("rmsnorm", {"prefix": p, "hidden_size": cfg.width, "eps": 1e-5})  # noqa: E731
    layer = lambda i: PartSpec("prenorm", {  # noqa: E731
        "prefix": f"l{i}.", "mixer": PartSpec("running_mean", {"prefix": "mix.", "hidden_size": cfg.width}),
        "feed_forward": PartSpec("swiglu", {"prefix": "ffn.", "hidden_size": cfg.width, "intermediate_size": 2 * cfg.width}),
        "mixer_norm": norm("n1."), "ffn_norm": norm("n2.")})
    return ModelSpec(architecture="ToyMeanForCausalLM", vocab_size=cfg.vocab, hidden_size=cfg.width, max_position=256,
                     embedding_name="emb", head_name=None, position=PartSpec("none", {}),
                     layers=tuple(layer(i) for i in range(cfg.depth)), final_norm=norm("nf."),
                     stop_token_ids=(cfg.stop,))


@pytest.mark.gpu
def test_another_architecture_runs_from_the_command_line_without_a_change_to_the_library(tmp_path, capsys):
    """An architecture with its own configuration class, its own config.json keys and a mixer with
    state, registered from here together with a named configuration: ``inference.py --model NAME
    --random-weights`` resolves it through the registry and generates; the same seed gives the
    same tokens, and they are the plain implementation's."""
    import json

    from simple_inference_autoresearch_b200 import config as config_module
    from simple_inference_autoresearch_b200 import inference

    MIXERS.register("running_mean")(RunningMeanMixer)
    registry.register_architecture("ToyMeanForCausalLM", ("toy_mean",), config_cls=ToyConfig, spec_builder=toy_mean_spec)
    path = tmp_path / "toy-mean.json"
    path.write_text(json.dumps(ToyConfig(32, 60, 2, 59).to_dict()))
    config_module.register_preset("toy-mean", path)
    try:
        args = ["--model", "toy-mean", "--random-weights", "--seed", "4", "--prompt-ids", "5,6,7,8", "--max-new-tokens", "6",
                "--temperature", "0", "--dtype", "float32", "--ignore-eos", "--no-cuda-graph"]
        # (the toy mixer is written in Python against the batch's host-side lists, which a captured step has not)
        assert inference.main(args) == 0
        first = capsys.readouterr().out.splitlines()[0]
        assert inference.main(args) == 0
        assert capsys.readouterr().out.splitlines()[0] == first
        tokens = [int(t) for t in first.split()]
        assert len(tokens) == 6
        # the plain model: running mean mixer + SwiGLU, greedy
        arch, cfg = registry.resolve_path(path)
        model = DecoderModel(arch.spec_builder(cfg), torch.float32, "cpu")
        w = random_tensors(model.tensor_specs(), 4, torch.bfloat16)
        w = {k: v.float() for k, v in w.items()}
        seq = [5, 6, 7, 8]
        for tok in tokens:
            x = w["emb"][torch.tensor(seq)]
            for i in range(2):
                p = f"l{i}."
                hn = plain_llama.rmsnorm(x, w[p + "n1.weight"], 1e-5)
                mean = torch.cumsum(hn, 0) / torch.arange(1, len(seq) + 1)[:, None]
                x = x + mean @ w[p + "mix.w"].T
                x = x + plain_llama.swiglu_mlp(plain_llama.rmsnorm(x, w[p + "n2.weight"], 1e-5), w, p + "ffn.")
            logits = plain_llama.rmsnorm(x, w["nf.weight"], 1e-5) @ w["emb"].T
            assert int(logits[-1].argmax()) == tok
            seq.append(tok)
    finally:
        MIXERS.unregister("running_mean")
        registry.unregister_architecture("ToyMeanForCausalLM")
        config_module._registered.pop("toy-mean", None)


def test_unknown_part_kind_is_a_clear_error():
    with pytest.raises(ValueError, match="unknown mixer kind 'nope'"):
        MIXERS.build(PartSpec("nope"))
    with pytest.raises(ValueError, match="already registered"):
        MIXERS.register("gqa_attention")(RunningMeanMixer)
