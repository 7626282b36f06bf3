"""Each part alone against the plain implementation's function for it, and what makes
the parts general: layers that differ inside one model, a windowed layer with pages
of its own, a run order that names a layer twice or lets a layer read another
layer's cache, a toy feed-forward with routing and a toy position encoding, and a toy mixer with per-request state that is registered, built and
stepped from here without touching the framework's files."""

import dataclasses

import pytest
import torch

from plain.plain_qwen3 import (plain_apply_rope, plain_embedding, plain_feed_forward, plain_gqa_attention,
                               plain_linear, plain_rms_norm, plain_rope_tables)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 3e-5, torch.bfloat16: 4e-2}


def _runtime(dtype):
    from quantinfer_b200.parts import Runtime
    return Runtime(dtype, DEV)


def _batch(lengths, starts, cache, want_all=True):
    """A StepBatch for entries of the given lengths at the given start positions."""
    from quantinfer_b200.engine.batch import StepEntry, batch_from_packed, pack_batch

    entries = [StepEntry(i, [0] * n, list(range(n)) if want_all else []) for i, n in enumerate(lengths)]
    slots = [cache.get(i).slot for i in range(len(lengths))]
    buf, layout, q_start, lens = pack_batch(entries, starts, slots, cache.host_tables, cache.max_blocks)
    dev = torch.from_numpy(buf).to(DEV)
    return batch_from_packed(dev, layout, entries, starts, slots, q_start, lens, len(cache.groups), cache.max_blocks)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from quantinfer_b200.config import NormSpec
    from quantinfer_b200.parts import build_part

    torch.manual_seed(0)
    spec = NormSpec(size=168, eps=2e-5, prefix="n.")
    part = build_part("norm", spec, _runtime(dtype))
    assert list(part.tensor_needs()) == ["n.weight"]
    gain = 1 + 0.1 * torch.randn(168)
    part.load({"n.weight": gain})
    resid, delta = torch.randn(5, 168), torch.randn(5, 168).to(dtype)
    r = resid.to(DEV)
    out = part.forward(r, delta.to(DEV))
    ref = plain_rms_norm(resid + delta.float(), gain, 2e-5)
    assert float((out.float().cpu() - ref).abs().max()) < TOL[dtype]
    assert float((r.cpu() - (resid + delta.float())).abs().max()) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from quantinfer_b200.config import FeedForwardSpec
    from quantinfer_b200.parts import build_part

    torch.manual_seed(1)
    spec = FeedForwardSpec(hidden_size=72, intermediate_size=136, prefix="m.")
    part = build_part("ffn", spec, _runtime(dtype))
    w = {"m.gate_proj.weight": (torch.randn(136, 72) * 0.1).to(dtype), "m.up_proj.weight": (torch.randn(136, 72) * 0.1).to(dtype),
         "m.down_proj.weight": (torch.randn(72, 136) * 0.1).to(dtype)}
    assert {k: v.shape for k, v in part.tensor_needs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    part.load(w)
    x = torch.randn(9, 72).to(dtype)
    y = part.forward(x.to(DEV))
    if y.dim() == 3:
        y = y.sum(0)
    ref = plain_feed_forward(x.float(), {k: v.float() for k, v in w.items()}, "m.")
    assert float((y.float().cpu() - ref).abs().max()) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("activation", ["gelu", "gelu_tanh", "relu"])
def test_the_gate_activation_is_a_parameter_of_the_feed_forward(dtype, activation):
    """The spec's `activation` reaches the kernel: the part alone against the formula, and a whole model
    (which the C++ driver runs) whose layers gate differently, stepped in portions, against the plain parts."""
    from quantinfer_b200.config import FeedForwardSpec, LayerSpec
    from quantinfer_b200.errors import ConfigError
    from quantinfer_b200.parts import build_part

    acts = {"gelu": lambda g: torch.nn.functional.gelu(g), "gelu_tanh": lambda g: torch.nn.functional.gelu(g, approximate="tanh"),
            "relu": torch.relu, "silu": lambda g: g / (1 + torch.exp(-g))}
    torch.manual_seed(2)
    spec = FeedForwardSpec(hidden_size=72, intermediate_size=136, activation=activation, prefix="m.")
    part = build_part("ffn", spec, _runtime(dtype))
    w = {"m.gate_proj.weight": (torch.randn(136, 72) * 0.3).to(dtype), "m.up_proj.weight": (torch.randn(136, 72) * 0.1).to(dtype),
         "m.down_proj.weight": (torch.randn(72, 136) * 0.1).to(dtype)}
    part.load(w)
    x = torch.randn(9, 72).to(dtype)
    y = part.forward(x.to(DEV))
    if y.dim() == 3:
        y = y.sum(0)
    f = {k: v.float() for k, v in w.items()}
    ref = (acts[activation](x.float() @ f["m.gate_proj.weight"].t()) * (x.float() @ f["m.up_proj.weight"].t())) @ f["m.down_proj.weight"].t()
    assert float((y.float().cpu() - ref).abs().max()) < TOL[dtype]
    with pytest.raises(ConfigError, match="no kernel"):
        build_part("ffn", FeedForwardSpec(72, 136, activation="swish7", prefix="m."), _runtime(dtype))
    if dtype != torch.float32:
        return
    # a model of two layers, the first gated by `activation`, the second by silu
    T = _SpecTools
    l0, l1 = T.layer(0), T.layer(1)
    l0 = LayerSpec(l0.mixer_norm, l0.mixer, l0.ffn_norm, dataclasses.replace(l0.ffn, activation=activation))
    spec = T.tiny_spec([l0, l1])
    eng, tensors = _engine(spec)
    assert eng.model.use_native
    ids = [int(t) for t in torch.randint(0, 97, (40,))]
    got = _run_in_portions(eng, ids, (25, 1, 1, 11, 2))
    assert eng.model.native, "the C++ driver should run a model of built-in parts"
    wf = {k: v.float() for k, v in tensors.items()}
    h = plain_embedding(wf["emb.weight"], ids)
    cos, sin = plain_rope_tables(1e4, 16, list(range(40)))
    for L in spec.layers:
        a, p = L.mixer, L.mixer.prefix
        n = plain_rms_norm(h, wf[L.mixer_norm.prefix + "weight"], L.mixer_norm.eps)
        q = plain_rms_norm(plain_linear(n, wf[p + "q_proj.weight"]).reshape(40, a.num_heads, 16), wf[p + "q_norm.weight"], a.qk_norm_eps)
        k = plain_rms_norm(plain_linear(n, wf[p + "k_proj.weight"]).reshape(40, a.num_kv_heads, 16), wf[p + "k_norm.weight"], a.qk_norm_eps)
        v = plain_linear(n, wf[p + "v_proj.weight"]).reshape(40, a.num_kv_heads, 16)
        att = plain_gqa_attention(plain_apply_rope(q, cos, sin), plain_apply_rope(k, cos, sin), v, None)
        h = h + plain_linear(att.reshape(40, a.num_heads * 16), wf[p + "o_proj.weight"])
        n = plain_rms_norm(h, wf[L.ffn_norm.prefix + "weight"], L.ffn_norm.eps)
        fp = L.ffn.prefix
        gate = acts[L.ffn.activation](plain_linear(n, wf[fp + "gate_proj.weight"]))
        h = h + plain_linear(gate * plain_linear(n, wf[fp + "up_proj.weight"]), wf[fp + "down_proj.weight"])
    ref = plain_linear(plain_rms_norm(h, wf["final.weight"], spec.final_norm.eps), wf["emb.weight"])
    assert float((got - ref).abs().max()) < 5e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    from quantinfer_b200.config import EmbeddingSpec, HeadSpec
    from quantinfer_b200.parts import build_part

    torch.manual_seed(2)
    rt = _runtime(dtype)
    emb = build_part("embedding", EmbeddingSpec(517, 40, "e."), rt)
    table = torch.randn(517, 40).to(dtype)
    emb.load({"e.weight": table})
    ids = [0, 516, 33]
    out = emb.forward(torch.tensor(ids, dtype=torch.int32, device=DEV))
    assert out.dtype == torch.float32 and torch.equal(out.cpu(), plain_embedding(table.float(), ids))
    tied = build_part("head", HeadSpec(517, 40, True, "h."), rt)
    assert tied.tensor_needs() == {}
    tied.tie(emb)
    x = torch.randn(3, 40).to(dtype)
    logits = tied.forward(x.to(DEV))
    assert logits.dtype == torch.float32
    assert float((logits.cpu() - plain_linear(x.float(), table.float())).abs().max()) < TOL[dtype] * 10
    untied = build_part("head", HeadSpec(517, 40, False, "h."), rt)
    assert list(untied.tensor_needs()) == ["h.weight"]


def _attention_weights(spec, dtype, sharp=3.0):
    d, nq, nkv, h = spec.head_dim, spec.num_heads, spec.num_kv_heads, spec.hidden_size
    p = spec.prefix
    return {p + "q_proj.weight": (torch.randn(nq * d, h) * 0.2).to(dtype), p + "k_proj.weight": (torch.randn(nkv * d, h) * 0.2).to(dtype),
            p + "v_proj.weight": (torch.randn(nkv * d, h) * 0.2).to(dtype), p + "o_proj.weight": (torch.randn(h, nq * d) * 0.2).to(dtype),
            # large q/k gains make the softmax peaked, so that one wrong key changes the output visibly
            p + "q_norm.weight": sharp * (1 + 0.1 * torch.randn(d)), p + "k_norm.weight": 1 + 0.1 * torch.randn(d)}


def _plain_attention(x, w, spec, window=None):
    p, d, nq, nkv = spec.prefix, spec.head_dim, spec.num_heads, spec.num_kv_heads
    T = x.shape[0]
    f = {k: v.float() for k, v in w.items()}
    q = plain_rms_norm(plain_linear(x, f[p + "q_proj.weight"]).reshape(T, nq, d), f[p + "q_norm.weight"], spec.qk_norm_eps)
    k = plain_rms_norm(plain_linear(x, f[p + "k_proj.weight"]).reshape(T, nkv, d), f[p + "k_norm.weight"], spec.qk_norm_eps)
    v = plain_linear(x, f[p + "v_proj.weight"]).reshape(T, nkv, d)
    cos, sin = plain_rope_tables(spec.position.theta, d, list(range(T)))
    a = plain_gqa_attention(plain_apply_rope(q, cos, sin), plain_apply_rope(k, cos, sin), v, window)
    return plain_linear(a.reshape(T, nq * d), f[p + "o_proj.weight"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq, nkv, d, window, page", [(4, 2, 16, None, 4), (6, 3, 48, None, 32), (4, 2, 64, None, 16),
                                                      (8, 1, 32, 11, 8), (4, 2, 64, 40, 16)])
def test_attention_part_in_portions(dtype, nq, nkv, d, window, page):
    """The mixer alone over a paged cache: one sequence fed in portions equals the plain
    whole-sequence attention, with a window and without."""
    from quantinfer_b200.cache import CacheManager
    from quantinfer_b200.config import AttentionSpec, PositionSpec
    from quantinfer_b200.parts import build_part

    torch.manual_seed(3)
    hidden, T = 56, 150
    spec = AttentionSpec(hidden, nq, nkv, d, PositionSpec(d, d, 30000.0, 256), qk_norm=True, qk_norm_eps=1e-5,
                         window=window, prefix="a.")
    rt = _runtime(dtype)
    part = build_part("mixer", spec, rt)
    w = _attention_weights(spec, dtype)
    part.load(w)
    cache = CacheManager([part.cache_need()], page, 64, 2, 256, dtype, DEV)
    cache.open(0)
    x = torch.randn(T, hidden).to(dtype)
    ref = _plain_attention(x.float(), w, spec, window)
    outs, pos = [], 0
    for n in (70, 1, 1, 2, 33, 1, 42):
        cache.prepare(0, n)
        batch = _batch([n], [pos], cache)
        y = part.forward(x[pos:pos + n].to(DEV), batch, cache.view(0))
        outs.append(y.sum(0) if y.dim() == 3 else y)
        cache.commit(0)
        pos += n
    got = torch.cat(outs).float().cpu()
    assert rt.status.item() == 0
    # bfloat16: values here reach |8|, where one bfloat16 step is 2^-5; six roundings of
    # intermediates feed a peaked softmax, so the bound is 2^-6 of the largest value
    tol = 1e-4 if dtype == torch.float32 else float(ref.abs().max()) * 2 ** -6
    assert float((got - ref).abs().max()) < tol
    if window:
        assert cache.free_pages() > 64 - -(-T // page)      # pages that the window passed went back


# ------------------------------------------------------------------ generality of the model

class _SpecTools:
    @staticmethod
    def tiny_spec(layers, order=None, hidden=48, vocab=97):
        from quantinfer_b200.config import (EmbeddingSpec, HeadSpec, LayerCall, ModelSpec, NormSpec)

        order = order or tuple(LayerCall(i, i) for i in range(len(layers)))
        return ModelSpec("Test", vocab, hidden, 128, EmbeddingSpec(vocab, hidden, "emb."), tuple(layers), tuple(order),
                         NormSpec(hidden, 1e-6, "final."), HeadSpec(vocab, hidden, True, "head."))

    @staticmethod
    def layer(i, hidden=48, nq=4, nkv=2, d=16, inter=80, window=None, mixer=None):
        from quantinfer_b200.config import AttentionSpec, FeedForwardSpec, LayerSpec, NormSpec, PositionSpec

        p = f"l{i}."
        mixer = mixer or AttentionSpec(hidden, nq, nkv, d, PositionSpec(d, d, 1e4, 128), qk_norm=True, window=window,
                                       prefix=p + "attn.")
        return LayerSpec(NormSpec(hidden, 1e-6, p + "n1."), mixer, NormSpec(hidden, 1e-6, p + "n2."),
                         FeedForwardSpec(hidden, inter, "silu", p + "mlp."))


def _engine(spec, dtype="float32", seed=0, max_tokens=512, **kw):
    from quantinfer_b200.engine import Engine, tensor_needs_of_spec
    from quantinfer_b200.weights import random_tensors

    tensors = random_tensors(tensor_needs_of_spec(spec), seed, torch.bfloat16)
    for k in tensors:
        if k.endswith("q_norm.weight"):
            tensors[k] = tensors[k] * 3.0
    return Engine(spec, tensors, dtype=dtype, page_size=8, max_tokens=max_tokens, max_requests=4, **kw), tensors


def _plain_model(tensors, spec, ids):
    """The plain forward pass for a spec built here: per call of the run order, the plain
    parts, with the cache-sharing rule (a reading layer uses the writer's keys and values)."""
    w = {k: v.float() for k, v in tensors.items()}
    h = plain_embedding(w["emb.weight"], ids)
    T = len(ids)
    kv = {}
    for call in spec.order:
        L = spec.layers[call.layer]
        a = L.mixer
        n = plain_rms_norm(h, w[L.mixer_norm.prefix + "weight"], L.mixer_norm.eps)
        p, d = a.prefix, a.head_dim
        q = plain_rms_norm(plain_linear(n, w[p + "q_proj.weight"]).reshape(T, a.num_heads, d), w[p + "q_norm.weight"], a.qk_norm_eps)
        cos, sin = plain_rope_tables(a.position.theta, d, list(range(T)))
        q = plain_apply_rope(q, cos, sin)
        if call.writes_cache:
            k = plain_rms_norm(plain_linear(n, w[p + "k_proj.weight"]).reshape(T, a.num_kv_heads, d), w[p + "k_norm.weight"], a.qk_norm_eps)
            kv[call.cache] = (plain_apply_rope(k, cos, sin), plain_linear(n, w[p + "v_proj.weight"]).reshape(T, a.num_kv_heads, d))
        k, v = kv[call.cache]
        att = plain_gqa_attention(q, k, v, a.window).reshape(T, a.num_heads * d)
        h = h + plain_linear(att, w[p + "o_proj.weight"])
        n = plain_rms_norm(h, w[L.ffn_norm.prefix + "weight"], L.ffn_norm.eps)
        h = h + plain_feed_forward(n, w, L.ffn.prefix)
    return plain_linear(plain_rms_norm(h, w["final.weight"], spec.final_norm.eps), w["emb.weight"])


def _run_in_portions(eng, ids, cuts):
    from quantinfer_b200.engine import StepEntry

    eng.open("r")
    rows, pos = [], 0
    for n in cuts:
        rows.append(eng.step([StepEntry("r", ids[pos:pos + n], list(range(n)))]).cpu())
        pos += n
    eng.close("r")
    eng.cache.check_invariants()
    return torch.cat(rows)


def test_layers_that_differ_and_a_windowed_group():
    """Layer 0: 4 heads of 16 with a window of 9; layer 1: 3 heads of 32, MQA, all keys; layer 2: as layer 0
    without window. The windowed layer gets a page group of its own and gives pages back."""
    T = _SpecTools
    layers = [T.layer(0, window=9), T.layer(1, nq=3, nkv=1, d=32, inter=56), T.layer(2, inter=100)]
    spec = T.tiny_spec(layers)
    eng, tensors = _engine(spec)
    assert len(eng.cache.groups) == 3
    ids = [int(x) for x in torch.randint(0, 97, (90,))]
    got = _run_in_portions(eng, ids, (40, 1, 1, 17, 2, 29))
    ref = _plain_model(tensors, spec, ids)
    assert float((got - ref).abs().max()) < 5e-5


def test_order_names_a_layer_twice_and_shares_a_cache():
    """Run order: layer 0, layer 1, layer 0 again (its weights reused, a cache entry of its own), then
    layer 2 reading the keys and values that the first call of layer 0 wrote."""
    from quantinfer_b200.config import LayerCall

    T = _SpecTools
    layers = [T.layer(0), T.layer(1, inter=56), T.layer(2)]
    order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(2, 0, writes_cache=False))
    spec = T.tiny_spec(layers, order)
    eng, tensors = _engine(spec)
    assert eng.spec.cache_entries() == 3 and len(eng.cache.groups) == 1
    ids = [int(x) for x in torch.randint(0, 97, (70,))]
    got = _run_in_portions(eng, ids, (33, 1, 1, 1, 30, 4))
    ref = _plain_model(tensors, spec, ids)
    assert float((got - ref).abs().max()) < 5e-5


def test_bad_run_orders_are_refused():
    from quantinfer_b200.config import LayerCall
    from quantinfer_b200.errors import ConfigError

    T = _SpecTools
    layers = [T.layer(0), T.layer(1)]
    for order in [(LayerCall(0, 0), LayerCall(1, 0)),                       # two writers of one entry
                  (LayerCall(0, 1, writes_cache=False), LayerCall(1, 1)),    # read before written
                  (LayerCall(0, 0), LayerCall(5, 1))]:                       # no such layer
        with pytest.raises(ConfigError):
            T.tiny_spec(layers, order).validate()
    # a reader whose mixer keeps something else than the writer
    spec = T.tiny_spec([T.layer(0), T.layer(1, nq=3, nkv=1, d=32)], (LayerCall(0, 0), LayerCall(1, 0, writes_cache=False)))
    with pytest.raises(ConfigError, match="keeps something else"):
        _engine(spec)


# ------------------------------------------------------------------ a toy mixer with state of its own

@dataclasses.dataclass(frozen=True)
class ToyStateSpec:
    hidden_size: int
    decay: float
    prefix: str = ""
    kind: str = "toy_running_mean"


def _register_toy():
    from quantinfer_b200.cache import StateNeed
    from quantinfer_b200.parts import Part, register_part
    from quantinfer_b200.weights import TensorNeed

    class ToyRunningMean(Part):
        """y_t = W (s_t), s_t = decay * s_{t-1} + x_t: a recurrence over the sequence whose state s lives
        in the request's slot. Written with torch operations on the batch's device arrays only (no host
        list, no synchronisation, shapes fixed by the batch's counts), so that it also runs inside a
        captured step: it is a test double, not a kernel."""

        @classmethod
        def needs_of_spec(cls, spec):
            return {spec.prefix + "mix.weight": TensorNeed((spec.hidden_size, spec.hidden_size))}

        def load(self, tensors):
            self.w = tensors[self.spec.prefix + "mix.weight"].to(self.runtime.device, torch.float32)

        def cache_need(self):
            return StateNeed((self.spec.hidden_size,), torch.float32)

        def forward(self, x, batch, cache):
            n, decay = x.shape[0], self.spec.decay
            xf = x.float()
            req, q0, slots = batch.token_req.long(), batch.q_start.long(), batch.slot_ids.long()
            local = torch.arange(n, device=x.device) - q0[req]            # place of a row within its entry
            gap = local[:, None] - local[None, :]
            earlier = (req[:, None] == req[None, :]) & (gap >= 0)
            weights = torch.where(earlier, torch.pow(decay, gap.clamp(min=0).float()), torch.zeros((), device=x.device))
            carried = torch.pow(decay, (local + 1).float())[:, None] * cache.state[slots[req]]
            s = weights @ xf + carried                                     # s_t for every row
            cache.state.index_copy_(0, slots, s[q0[1:] - 1])              # each entry's last row is its new state
            return (s @ self.w.t()).to(x.dtype)

    register_part("mixer", "toy_running_mean", ToyRunningMean)


def _toy_state_engine(**kw):
    _register_toy()
    T = _SpecTools
    layers = [T.layer(0), T.layer(1, mixer=ToyStateSpec(48, 0.9, "l1.toy.")), T.layer(2)]
    return _engine(T.tiny_spec(layers), **kw)


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    from quantinfer_b200.engine import StepEntry

    eng, tensors = _toy_state_engine(use_graphs=False)
    assert "l1.toy.mix.weight" in tensors and len(eng.cache.groups) == 1 and list(eng.cache.states) == [1]
    ids_a = [int(x) for x in torch.randint(0, 97, (40,))]
    ids_b = [int(x) for x in torch.randint(0, 97, (25,))]

    def whole(ids):
        eng.open("w")
        out = eng.step([StepEntry("w", ids, list(range(len(ids))))]).cpu()
        eng.close("w")
        return out

    ref_a, ref_b = whole(ids_a), whole(ids_b)
    # the recurrence, token by token on the host, against the part's one-pass form
    x = torch.randn(7, 48)
    s, rows = torch.zeros(48), []
    for t in range(7):
        s = 0.9 * s + x[t]
        rows.append(s)
    eng.open("p")
    from quantinfer_b200.engine.batch import StepEntry as _E
    batch = eng.make_batch([_E("p", [0] * 7, [])])
    mixer = eng.model.blocks[1].mixer
    got = mixer.forward(x.to(DEV), batch, eng._views[1]).cpu()
    eng.close("p")
    assert float((got - torch.stack(rows) @ tensors["l1.toy.mix.weight"].float().t()).abs().max()) < 1e-5
    # the same two requests interleaved in portions; slots are reused, so a state that
    # was not reset at open or that leaked between requests would show
    eng.open("a"), eng.open("b")
    got_a, got_b = [], []
    got_a.append(eng.step([StepEntry("a", ids_a[:10], list(range(10)))]).cpu())
    out = eng.step([StepEntry("a", ids_a[10:11], [0]), StepEntry("b", ids_b[:20], list(range(20)))]).cpu()
    got_a.append(out[:1]), got_b.append(out[1:])
    out = eng.step([StepEntry("b", ids_b[20:], list(range(5))), StepEntry("a", ids_a[11:], list(range(29)))]).cpu()
    got_b.append(out[:5]), got_a.append(out[5:])
    eng.close("a"), eng.close("b")
    assert float((torch.cat(got_a) - ref_a).abs().max()) < 2e-5
    assert float((torch.cat(got_b) - ref_b).abs().max()) < 2e-5
    assert not torch.allclose(ref_a[5], whole(ids_a[5:])[0])       # the recurrence does depend on its past


def test_toy_mixer_with_state_in_captured_steps_and_steps_that_run_ahead():
    """The stateful mixer under CUDA graphs: decode steps of one batch size are one captured graph,
    replayed for other requests in other slots and in another order of slots; and through the scheduler
    with steps launched ahead of the host. Both against the same engine without graphs."""
    import quantinfer_b200
    from quantinfer_b200.engine import StepEntry
    from quantinfer_b200.errors import QuantInferError

    prompts = {k: [int(x) for x in torch.randint(0, 97, (n,))] for k, n in (("a", 9), ("b", 21), ("c", 14), ("d", 5))}
    feed = [int(x) for x in torch.randint(0, 97, (12,))]

    def script(eng):
        rows, slots = [], []
        for pair in (("a", "b"), ("c", "d")):        # the second pair takes the first pair's slots, the other way round
            for rid in pair:
                eng.open(rid)
                rows.append(eng.step([StepEntry(rid, prompts[rid], [len(prompts[rid]) - 1])]).cpu())
            slots.append([eng.cache.get(rid).slot for rid in pair])
            for t in feed:
                rows.append(eng.step([StepEntry(rid, [t], [0]) for rid in pair]).cpu())
            for rid in pair:
                eng.close(rid)
        return torch.cat(rows), slots

    plain_eng, _ = _toy_state_engine(use_graphs=False)
    graph_eng, _ = _toy_state_engine(use_graphs=True)
    ref, _ = script(plain_eng)
    got, slots = script(graph_eng)
    assert slots[0] == slots[1][::-1]                                  # same slots, other order
    assert len(graph_eng._graphs) == 1                                 # every decode step of both pairs replayed one graph
    assert float((got - ref).abs().max()) < 1e-5
    # a part that reads the host-side lists in such a step is told so
    g = next(iter(graph_eng._graphs.values()))
    with pytest.raises(QuantInferError, match="on the device"):
        g["batch"].h_slot_ids[0]
    # through the scheduler: four prompts on two sequence slots, steps that run ahead
    outs = []
    for eng, ahead in ((plain_eng, False), (graph_eng, True)):
        m = quantinfer_b200.Model.from_engine(eng, max_batch_tokens=32, run_ahead=ahead)
        outs.append(m.generate_batch(list(prompts.values()), max_new_tokens=20, eos_token_id=None))
        if ahead:
            assert m.last_scheduler.steps_ahead > 10
        eng.cache.check_invariants()
    assert outs[0] == outs[1]


def test_state_of_fixed_size_is_rolled_back_when_a_step_fails():
    """A step that fails gives a request's fixed-size state back as it was: once when a second request of
    the step finds no page (nothing ran), once when a kernel flags a block table entry that holds no page
    (the layers after it ran, and the stateful mixer overwrote its state). The request then goes on and
    equals the run that never failed."""
    from quantinfer_b200.engine import StepEntry
    from quantinfer_b200.errors import OutOfPages, QuantInferError

    eng, _ = _toy_state_engine(use_graphs=False, max_tokens=64)      # eight pages of eight positions
    ids = [int(x) for x in torch.randint(0, 97, (30,))]
    eng.open("w")
    ref = eng.step([StepEntry("w", ids, list(range(30)))]).cpu()
    eng.close("w")
    eng.open("r"), eng.open("big")
    rows = [eng.step([StepEntry("r", ids[:12], list(range(12)))]).cpu()]
    state = eng.cache.states[1][eng.cache.get("r").slot].clone()
    with pytest.raises(OutOfPages):          # r holds two pages and takes a third; the second entry wants eight
        eng.step([StepEntry("r", ids[12:20], list(range(8))), StepEntry("big", [1] * 60, [])])
    eng.cache.check_invariants()
    assert eng.length("r") == 12 and torch.equal(eng.cache.states[1][eng.cache.get("r").slot], state)
    # a block table entry without a page: the attention kernels set the status bit and skip the access
    slot = eng.cache.get("r").slot
    page = int(eng.cache.host_tables[0][slot, 0])
    eng.cache.host_tables[0][slot, 0] = -1
    with pytest.raises(QuantInferError, match="cache page"):
        eng.step([StepEntry("r", ids[12:20], list(range(8)))])
    eng.cache.host_tables[0][slot, 0] = page
    assert eng.length("r") == 12 and torch.equal(eng.cache.states[1][slot], state)
    rows.append(eng.step([StepEntry("r", ids[12:20], list(range(8)))]).cpu())
    rows.append(eng.step([StepEntry("r", ids[20:], list(range(10)))]).cpu())
    eng.close("r"), eng.close("big")
    eng.cache.check_invariants()
    assert float((torch.cat(rows) - ref).abs().max()) < 2e-5


# ------------------------------------------------------------------ a toy feed-forward with routing, another position encoding

@dataclasses.dataclass(frozen=True)
class ToyRoutedSpec:
    hidden_size: int
    experts: int
    prefix: str = ""
    kind: str = "toy_top1_experts"


@dataclasses.dataclass(frozen=True)
class ToyAnglesSpec:
    head_dim: int
    rotary_dim: int
    step: float
    max_positions: int
    kind: str = "toy_linear_angles"


def _register_toy_ffn_and_position():
    from quantinfer_b200.parts import Part, register_part
    from quantinfer_b200.weights import TensorNeed

    class ToyTop1Experts(Part):
        """y = p_e * W_e x with e = argmax of the router's 32-bit logits and p its softmax: every token
        takes one of `experts` small matrices. Written with torch operations: a test double."""

        @classmethod
        def needs_of_spec(cls, spec):
            h, p = spec.hidden_size, spec.prefix
            needs = {p + "router.weight": TensorNeed((spec.experts, h))}
            for e in range(spec.experts):
                needs[p + f"expert{e}.weight"] = TensorNeed((h, h))
            return needs

        def load(self, tensors):
            p, dev = self.spec.prefix, self.runtime.device
            self.router = tensors[p + "router.weight"].to(dev, torch.float32)
            self.experts = torch.stack([tensors[p + f"expert{e}.weight"].to(dev, torch.float32) for e in range(self.spec.experts)])

        def forward(self, x):
            logits = x.float() @ self.router.t()
            prob, which = torch.softmax(logits, dim=-1).max(dim=-1)
            y = torch.einsum("nh,nkh->nk", x.float(), self.experts[which]) * prob[:, None]
            return y.to(x.dtype)

    class ToyLinearAngles(Part):
        """Pair p of a head turns by position * step * (p + 1): the mixer's interface to a position
        encoding is its cos/sin table [positions, rotary_dim / 2] and `rotary_dim`."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.rotary_dim = spec.rotary_dim
            ang = _toy_angles(spec, range(spec.max_positions)).to(runtime.device)
            self.cos, self.sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()

    register_part("ffn", "toy_top1_experts", ToyTop1Experts)
    register_part("position", "toy_linear_angles", ToyLinearAngles)


def _toy_angles(spec, positions):
    pos = torch.tensor(list(positions), dtype=torch.float32)
    return pos[:, None] * (spec.step * torch.arange(1, spec.rotary_dim // 2 + 1, dtype=torch.float32))[None, :]


def test_toy_feed_forward_with_routing_and_another_position_encoding():
    """Layer 1 has a routed feed-forward and layer 2 a position encoding of its own, both registered
    here; the model is built from the spec and stepped in portions, against the plain parts."""
    from quantinfer_b200.config import AttentionSpec, LayerSpec, NormSpec
    from plain.plain_qwen3 import plain_apply_rope

    _register_toy_ffn_and_position()
    T = _SpecTools
    hidden, d = 48, 16
    pos2 = ToyAnglesSpec(d, d, 0.013, 128)
    l1 = T.layer(1)
    l1 = LayerSpec(l1.mixer_norm, l1.mixer, l1.ffn_norm, ToyRoutedSpec(hidden, 3, "l1.moe."))
    l2 = T.layer(2, mixer=AttentionSpec(hidden, 4, 2, d, pos2, qk_norm=True, window=None, prefix="l2.attn."))
    spec = T.tiny_spec([T.layer(0), l1, l2])
    eng, tensors = _engine(spec)
    assert "l1.moe.router.weight" in tensors and "l1.moe.expert2.weight" in tensors
    ids = [int(x) for x in torch.randint(0, 97, (60,))]
    got = _run_in_portions(eng, ids, (21, 1, 1, 30, 2, 5))

    w = {k: v.float() for k, v in tensors.items()}
    h = plain_embedding(w["emb.weight"], ids)
    n_tok = len(ids)
    used = set()
    for i, L in enumerate(spec.layers):
        a = L.mixer
        n = plain_rms_norm(h, w[L.mixer_norm.prefix + "weight"], L.mixer_norm.eps)
        p = a.prefix
        if a.position.kind == "toy_linear_angles":
            ang = _toy_angles(a.position, range(n_tok))
            cos, sin = torch.cos(ang), torch.sin(ang)
        else:
            cos, sin = plain_rope_tables(a.position.theta, d, list(range(n_tok)))
        q = plain_rms_norm(plain_linear(n, w[p + "q_proj.weight"]).reshape(n_tok, a.num_heads, d), w[p + "q_norm.weight"], a.qk_norm_eps)
        k = plain_rms_norm(plain_linear(n, w[p + "k_proj.weight"]).reshape(n_tok, a.num_kv_heads, d), w[p + "k_norm.weight"], a.qk_norm_eps)
        v = plain_linear(n, w[p + "v_proj.weight"]).reshape(n_tok, a.num_kv_heads, d)
        att = plain_gqa_attention(plain_apply_rope(q, cos, sin), plain_apply_rope(k, cos, sin), v, None).reshape(n_tok, a.num_heads * d)
        h = h + plain_linear(att, w[p + "o_proj.weight"])
        n = plain_rms_norm(h, w[L.ffn_norm.prefix + "weight"], L.ffn_norm.eps)
        if L.ffn.kind == "toy_top1_experts":
            fp = L.ffn.prefix
            prob, which = torch.softmax(n @ w[fp + "router.weight"].t(), dim=-1).max(dim=-1)
            used |= set(which.tolist())
            h = h + torch.stack([w[fp + f"expert{int(e)}.weight"] @ n[t] for t, e in enumerate(which)]) * prob[:, None]
        else:
            h = h + plain_feed_forward(n, w, L.ffn.prefix)
    ref = plain_linear(plain_rms_norm(h, w["final.weight"], spec.final_norm.eps), w["emb.weight"])
    assert len(used) > 1, "the router sent every token to one expert: the test shows nothing"
    assert float((got - ref).abs().max()) < 5e-5


@dataclasses.dataclass(frozen=True)
class ToyScaledEmbeddingSpec:
    vocab_size: int
    hidden_size: int
    scale: float
    prefix: str = ""
    kind: str = "toy_scaled_embedding"


@dataclasses.dataclass(frozen=True)
class ToySoftcapHeadSpec:
    vocab_size: int
    hidden_size: int
    cap: float
    tied: bool = False
    prefix: str = ""
    kind: str = "toy_softcap_head"


def test_a_scaled_embedding_and_a_capped_head_are_parts_too():
    """What stands before the first block and after the last norm are parts of their own categories: an
    embedding that scales its rows and a head that soft-caps its logits are registered here and named by
    the model's spec; nothing in the model's forward pass changes. (Test doubles in torch.)"""
    from quantinfer_b200.parts import Part, register_part
    from quantinfer_b200.weights import TensorNeed

    class ToyScaledEmbedding(Part):
        @classmethod
        def needs_of_spec(cls, spec):
            return {spec.prefix + "weight": TensorNeed((spec.vocab_size, spec.hidden_size), "table")}

        def load(self, tensors):
            self.table = tensors[self.spec.prefix + "weight"].to(self.runtime.device, torch.float32)

        def forward(self, token_ids):
            return (self.table[token_ids.long()] * self.spec.scale).contiguous()

        __call__ = forward

    class ToySoftcapHead(Part):
        @classmethod
        def needs_of_spec(cls, spec):
            return {spec.prefix + "weight": TensorNeed((spec.vocab_size, spec.hidden_size))}

        def load(self, tensors):
            self.w = tensors[self.spec.prefix + "weight"].to(self.runtime.device, torch.float32)

        def forward(self, x):
            return (self.spec.cap * torch.tanh((x.float() @ self.w.t()) / self.spec.cap)).contiguous()

        __call__ = forward

    register_part("embedding", "toy_scaled_embedding", ToyScaledEmbedding)
    register_part("head", "toy_softcap_head", ToySoftcapHead)
    T = _SpecTools
    base = T.tiny_spec([T.layer(0), T.layer(1)])
    spec = dataclasses.replace(base, embedding=ToyScaledEmbeddingSpec(97, 48, 6.9, "emb."), head=ToySoftcapHeadSpec(97, 48, 0.5, prefix="head."))
    eng, tensors = _engine(spec)
    assert "head.weight" in tensors
    ids = [int(t) for t in torch.randint(0, 97, (30,))]
    got = _run_in_portions(eng, ids, (19, 1, 1, 9))
    assert not eng.model.native                       # a part from outside: the parts' own forward runs
    w = {k: v.float() for k, v in tensors.items()}
    h = w["emb.weight"][ids] * 6.9
    cos, sin = plain_rope_tables(1e4, 16, list(range(30)))
    for L in spec.layers:
        a, p = L.mixer, L.mixer.prefix
        n = plain_rms_norm(h, w[L.mixer_norm.prefix + "weight"], L.mixer_norm.eps)
        q = plain_rms_norm(plain_linear(n, w[p + "q_proj.weight"]).reshape(30, a.num_heads, 16), w[p + "q_norm.weight"], a.qk_norm_eps)
        k = plain_rms_norm(plain_linear(n, w[p + "k_proj.weight"]).reshape(30, a.num_kv_heads, 16), w[p + "k_norm.weight"], a.qk_norm_eps)
        v = plain_linear(n, w[p + "v_proj.weight"]).reshape(30, a.num_kv_heads, 16)
        att = plain_gqa_attention(plain_apply_rope(q, cos, sin), plain_apply_rope(k, cos, sin), v, None)
        h = h + plain_linear(att.reshape(30, a.num_heads * 16), w[p + "o_proj.weight"])
        h = h + plain_feed_forward(plain_rms_norm(h, w[L.ffn_norm.prefix + "weight"], L.ffn_norm.eps), w, L.ffn.prefix)
    ref = 0.5 * torch.tanh(plain_linear(plain_rms_norm(h, w["final.weight"], spec.final_norm.eps), w["head.weight"]) / 0.5)
    assert float((got - ref).abs().max()) < 5e-5
    assert float(ref.abs().max()) > 0.25                # the cap does bend these logits


def _rotate_interleaved(x, cos, sin, rot):
    """Pairs (2p, 2p + 1) of the first `rot` elements of each head turn by the angle of pair p; the rest
    passes. x [tokens, heads, d]; cos, sin [tokens, rot / 2]."""
    out = x.clone()
    a, b = x[..., 0:rot:2], x[..., 1:rot:2]
    c, s_ = cos[:, None, :], sin[:, None, :]
    out[..., 0:rot:2] = a * c - b * s_
    out[..., 1:rot:2] = a * s_ + b * c
    return out


@pytest.mark.parametrize("dtype, d, rot, n_tok", [("float32", 16, 16, 50), ("float32", 24, 12, 50), ("bfloat16", 128, 128, 300)])
def test_interleaved_pairs_are_a_parameter_of_the_position_encoding(dtype, d, rot, n_tok):
    """A position spec with pairing "interleaved" (and, in one case, a rotation over half the head): the
    mixer's kernels pair (2p, 2p + 1). In bfloat16 at head size 128 with a prompt of 300 tokens the fused
    projection and the fused decode attention, which only know the half-split rule, are passed over."""
    from quantinfer_b200.config import AttentionSpec, PositionSpec

    T = _SpecTools
    hidden = 64
    pos = PositionSpec(d, rot, 1e4, 512, pairing="interleaved")
    layers = [T.layer(i, hidden=hidden, mixer=AttentionSpec(hidden, 2, 1, d, pos, qk_norm=True, prefix=f"l{i}.attn.")) for i in range(2)]
    from quantinfer_b200.config import EmbeddingSpec, HeadSpec, LayerCall, ModelSpec, NormSpec
    spec = ModelSpec("Test", 97, hidden, 512, EmbeddingSpec(97, hidden, "emb."), tuple(layers),
                     (LayerCall(0, 0), LayerCall(1, 1)), NormSpec(hidden, 1e-6, "final."), HeadSpec(97, hidden, True, "head."))
    eng, tensors = _engine(spec, dtype=dtype, max_tokens=1024)
    ids = [int(x) for x in torch.randint(0, 97, (n_tok,))]
    cuts = (n_tok - 9, 1, 1, 5, 2)
    got = _run_in_portions(eng, ids, cuts)

    w = {k: v.float() for k, v in tensors.items()}
    h = plain_embedding(w["emb.weight"], ids)
    cos, sin = plain_rope_tables(1e4, rot, list(range(n_tok)))
    for L in spec.layers:
        a, p = L.mixer, L.mixer.prefix
        n = plain_rms_norm(h, w[L.mixer_norm.prefix + "weight"], L.mixer_norm.eps)
        q = plain_rms_norm(plain_linear(n, w[p + "q_proj.weight"]).reshape(n_tok, a.num_heads, d), w[p + "q_norm.weight"], a.qk_norm_eps)
        k = plain_rms_norm(plain_linear(n, w[p + "k_proj.weight"]).reshape(n_tok, a.num_kv_heads, d), w[p + "k_norm.weight"], a.qk_norm_eps)
        v = plain_linear(n, w[p + "v_proj.weight"]).reshape(n_tok, a.num_kv_heads, d)
        att = plain_gqa_attention(_rotate_interleaved(q, cos, sin, rot), _rotate_interleaved(k, cos, sin, rot), v, None)
        h = h + plain_linear(att.reshape(n_tok, a.num_heads * d), w[p + "o_proj.weight"])
        n = plain_rms_norm(h, w[L.ffn_norm.prefix + "weight"], L.ffn_norm.eps)
        h = h + plain_feed_forward(n, w, L.ffn.prefix)
    ref = plain_linear(plain_rms_norm(h, w["final.weight"], spec.final_norm.eps), w["emb.weight"])
    assert float((got - ref).abs().max()) < (5e-5 if dtype == "float32" else 4e-2)
    # the half-split rule on the same weights gives other logits: the parameter does reach the kernel
    half = dataclasses.replace(pos, pairing="half_split")
    spec_h = dataclasses.replace(spec, layers=tuple(dataclasses.replace(L, mixer=dataclasses.replace(L.mixer, position=half)) for L in layers))
    eng_h, _ = _engine(spec_h, dtype=dtype, max_tokens=1024)
    other = _run_in_portions(eng_h, ids, cuts)
    assert float((other - ref).abs().max()) > 10 * (5e-5 if dtype == "float32" else 4e-2)


@dataclasses.dataclass(frozen=True)
class ToyCenteredNormSpec:
    size: int
    eps: float
    prefix: str = ""
    kind: str = "toy_centered_norm"


def test_a_toy_norm_takes_partial_sums_through_the_documented_contract():
    """Another norm kind (mean removed, then scaled), registered here, in a bfloat16 model whose
    projections hand K-split partial sums to the norm that follows: the norm adds them with the
    package's helper and needs no kernel of its own for them."""
    from quantinfer_b200.config import LayerSpec
    from quantinfer_b200.parts import Part, register_part
    from quantinfer_b200.parts.norm import sum_partials
    from quantinfer_b200.weights import TensorNeed

    seen = {"partials": 0, "whole": 0}

    class ToyCenteredNorm(Part):
        @classmethod
        def needs_of_spec(cls, spec):
            return {spec.prefix + "weight": TensorNeed((spec.size,), "gain", "gain")}

        def load(self, tensors):
            self.gain = self._gain(tensors[self.spec.prefix + "weight"])

        def forward(self, resid, delta, rows=None, write_resid=True):
            if delta is not None:
                seen["partials" if delta.dim() == 3 else "whole"] += 1
                x = resid + sum_partials(delta).float()
                if write_resid and rows is None:
                    resid.copy_(x)
            else:
                x = resid
            if rows is not None:
                x = x[rows.long()]
            x = x - x.mean(dim=-1, keepdim=True)
            y = x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + self.spec.eps) * self.gain
            return y.to(self.runtime.dtype)

        __call__ = forward

    register_part("norm", "toy_centered_norm", ToyCenteredNorm)
    T = _SpecTools
    hidden = 128     # a product is cut along K from 1,024 up: the output projection (8 heads of 128) and the down projection
    base = [T.layer(i, hidden=hidden, nq=8, nkv=2, d=128, inter=1024) for i in range(2)]
    layers = [LayerSpec(base[0].mixer_norm, base[0].mixer, ToyCenteredNormSpec(hidden, 1e-5, "l0.n2."), base[0].ffn),
              LayerSpec(ToyCenteredNormSpec(hidden, 1e-5, "l1.n1."), base[1].mixer, base[1].ffn_norm, base[1].ffn)]
    spec = T.tiny_spec(layers, hidden=hidden)
    eng, tensors = _engine(spec, dtype="bfloat16", use_graphs=False)
    ids = [int(x) for x in torch.randint(0, 97, (40,))]
    got = _run_in_portions(eng, ids, (30, 1, 1, 1, 7))
    assert seen["partials"] > 0, "no projection of this model was cut along K: the test shows nothing"

    w = {k: v.float() for k, v in tensors.items()}
    h = plain_embedding(w["emb.weight"], ids)
    n_tok, d = len(ids), 128

    def norm(x, ns):
        if ns.kind == "rmsnorm":
            return plain_rms_norm(x, w[ns.prefix + "weight"], ns.eps)
        x = x - x.mean(dim=-1, keepdim=True)
        return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + ns.eps) * w[ns.prefix + "weight"]

    cos, sin = plain_rope_tables(1e4, d, list(range(n_tok)))
    for L in spec.layers:
        a, p = L.mixer, L.mixer.prefix
        n = norm(h, L.mixer_norm)
        q = plain_rms_norm(plain_linear(n, w[p + "q_proj.weight"]).reshape(n_tok, a.num_heads, d), w[p + "q_norm.weight"], a.qk_norm_eps)
        k = plain_rms_norm(plain_linear(n, w[p + "k_proj.weight"]).reshape(n_tok, a.num_kv_heads, d), w[p + "k_norm.weight"], a.qk_norm_eps)
        v = plain_linear(n, w[p + "v_proj.weight"]).reshape(n_tok, a.num_kv_heads, d)
        att = plain_gqa_attention(plain_apply_rope(q, cos, sin), plain_apply_rope(k, cos, sin), v, None)
        h = h + plain_linear(att.reshape(n_tok, a.num_heads * d), w[p + "o_proj.weight"])
        h = h + plain_feed_forward(norm(h, L.ffn_norm), w, L.ffn.prefix)
    ref = plain_linear(plain_rms_norm(h, w["final.weight"], spec.final_norm.eps), w["emb.weight"])
    assert float((got - ref).abs().max()) < 4e-2


def test_shared_cache_and_window_through_the_tensor_core_kernels():
    """The run order that shares a cache entry and a windowed layer, at head size 64 in bfloat16: the
    attention kernels of the serving path (the decode kernel makes its own queries and, for the layer
    that writes, the new key and value; the reading layer writes nothing), single tokens included."""
    from quantinfer_b200.config import LayerCall

    T = _SpecTools
    ids = [int(x) for x in torch.randint(0, 97, (120,))]
    layers = [T.layer(0, d=64), T.layer(1, d=64, inter=56), T.layer(2, d=64)]
    order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(2, 0, writes_cache=False))
    spec = T.tiny_spec(layers, order)
    eng, tensors = _engine(spec, dtype="bfloat16")
    got = _run_in_portions(eng, ids, (33, 1, 1, 1, 30, 4) + (1,) * 50)
    assert float((got - _plain_model(tensors, spec, ids)).abs().max()) < 3e-2
    spec = T.tiny_spec([T.layer(0, d=64, window=24), T.layer(1, nkv=1, d=64, inter=56)])
    eng, tensors = _engine(spec, dtype="bfloat16")
    got = _run_in_portions(eng, ids, (40, 1, 1, 17, 2) + (1,) * 59)
    assert float((got - _plain_model(tensors, spec, ids)).abs().max()) < 3e-2
