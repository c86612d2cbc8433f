"""The Sokolorn decoder: its mechanisms one by one against `plain_sokolorn`, then whole models through the
engine's step function, scheduler and entry points.  The plain implementation shares nothing with the
package; it runs in float64 on bfloat16-rounded random weights."""
import math

import pytest
import torch

import plain_sokolorn as plain
import sokolorn_models
from helpers import assert_close, engine_model, run_portions, run_whole, write_model_folder

BF16 = dict(rmse=0.12, max=0.4, cosine=0.993)


def tokens_for(config, count, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, config["vocab"], (count,), generator=g).tolist()


def plain_logits(config, weights, tokens):
    return plain.forward(config, {k: v.double() for k, v in weights.items()}, tokens).float()


# ----------------------------------------------------------------------------- without a GPU
def test_config_and_plan_name_every_tensor():
    from mini_llm_runtime_b200 import models  # noqa: F401
    from mini_llm_runtime_b200.config.registry import config_from_dict, plan_for
    from mini_llm_runtime_b200.engine.structure import expected_weights
    for name in sokolorn_models.ALL:
        config = sokolorn_models.get(name)
        weights = sokolorn_models.random_weights(config, 1)
        plan = plan_for(config_from_dict(config))
        expected = expected_weights(plan)
        assert set(expected) == set(weights), name
        for key, spec in expected.items():
            assert tuple(spec.shape) == tuple(weights[key].shape), key
        for i, (layer, run) in enumerate(zip(config["layers"], plan.schedule)):
            assert run.kv_from == layer["mixer"].get("kv_from"), (name, i)


@pytest.mark.parametrize("path,value,message", [
    (("width",), None, "width"),
    (("norm", "eps"), None, "eps"),
    (("layers", 0, "type"), "lightning", "attention_2"),
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "rot"), {"base": 10.0, "dims": 4}, "attention_2"),
    (("layers", 3, "mixer", "kv_from"), 0, "differ"),
    (("layers", 1, "mixer", "mask"), {"size": 4}, "'attention'"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "dims"),
    (("layers", 1, "mixer", "rot", "scaling", "high"), 0.5, "high"),
    (("layers", 2, "mixer", "kv_from"), 0, "kv_from"),
    (("layers", 2, "mixer", "kv_from"), 2, "earlier"),
    (("layers", 2, "mixer", "vdim"), 8, "differ"),
    (("layers", 1, "mlp", "router", "top"), 9, "top"),
    (("layers", 1, "mlp", "expert"), None, "expert"),
    (("layers", 0, "mlp", "kind"), "gated", "dense"),
    (("layers", 0, "mlp", "ff"), None, "ff"),
])
def test_config_errors_name_the_key(path, value, message):
    from mini_llm_runtime_b200 import models  # noqa: F401
    from mini_llm_runtime_b200.config.base import ConfigError
    from mini_llm_runtime_b200.config.registry import config_from_dict
    config = sokolorn_models.get("small_a")
    at = config
    for key in path[:-1]:
        at = at[key]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        config_from_dict(config)


def test_plain_window_sees_itself_and_the_tokens_before_it():
    seen = plain.visible(12, 4)
    assert seen[11].tolist() == [False] * 8 + [True] * 4
    assert seen[2].tolist() == [True] * 3 + [False] * 9
    assert plain.visible(5, 1)[4].tolist() == [False] * 4 + [True]
    assert plain.visible(5, None)[4].all()


def test_plain_sink_counts_once_is_not_scaled_and_has_no_value():
    scores = torch.zeros(1, 1, 3, dtype=torch.float64)
    seen = torch.ones(1, 3, dtype=torch.bool)
    p = plain.softmax_with_sink(scores, seen, torch.tensor([math.log(3.0)], dtype=torch.float64))
    assert torch.allclose(p, torch.full((1, 1, 3), 1.0 / 6.0, dtype=torch.float64))
    q = torch.zeros(1, 1, 2, dtype=torch.float64)
    k = torch.zeros(1, 1, 2, dtype=torch.float64)
    v = torch.tensor([[[5.0]]], dtype=torch.float64)
    out = plain.attend(q, k, v, 123.0, plain.visible(1, None), torch.tensor([0.0], dtype=torch.float64))
    assert torch.allclose(out, torch.tensor([[[2.5]]], dtype=torch.float64))       # half the weight went to the sink, whatever the scale


def test_plain_rotation_turns_halves_and_keeps_the_rest():
    x = torch.arange(1.0, 7.0, dtype=torch.float64).view(1, 1, 6)
    y = plain.rotate_halves(x, torch.tensor([3]), [0.5, 0.25])
    for i, f in enumerate([0.5, 0.25]):
        a = 3 * f
        assert math.isclose(float(y[0, 0, i]), float(x[0, 0, i]) * math.cos(a) - float(x[0, 0, i + 2]) * math.sin(a))
        assert math.isclose(float(y[0, 0, i + 2]), float(x[0, 0, i + 2]) * math.cos(a) + float(x[0, 0, i]) * math.sin(a))
    assert y[0, 0, 4:].tolist() == [5.0, 6.0]
    assert torch.equal(plain.rotate_halves(x, torch.tensor([0]), [0.5, 0.25]), x)


def test_plain_frequency_scaling_keeps_short_waves_slows_long_ones_and_blends_between():
    base, dims = 100.0, 8
    plainf = plain.scaled_frequencies(base, dims, None)
    f = plain.scaled_frequencies(base, dims, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64})
    assert f[0] == plainf[0] == 1.0                                       # wavelength 6.3 < 16
    assert math.isclose(f[3], plainf[3] / 8.0)                            # wavelength 199 > 64
    for i in (1, 2):                                                      # wavelengths 19.9 and 62.8 lie between
        s = (64 * plainf[i] / (2 * math.pi) - 1.0) / 3.0
        assert 0.0 < s < 1.0 and math.isclose(f[i], (1 - s) * plainf[i] / 8.0 + s * plainf[i])
    from mini_llm_runtime_b200.parts.rotary import scaled_frequencies
    import numpy as np
    assert np.allclose(scaled_frequencies(np.array(plainf), 8.0, 1.0, 4.0, 64.0), np.array(f), rtol=1e-12)


def test_plain_expert_clamps_the_gate_above_and_the_other_on_both_sides():
    w = {"gate": torch.eye(3, dtype=torch.float64), "up": torch.eye(3, dtype=torch.float64), "down": torch.eye(3, dtype=torch.float64)}
    h = torch.tensor([[5.0, -5.0, 0.5]], dtype=torch.float64)
    y = plain.clamped_expert(h, w, "", 1.0)[0]
    sig = lambda z: 1.0 / (1.0 + math.exp(-z))
    assert math.isclose(float(y[0]), 1.0 * sig(1.702) * 2.0)                 # gate cut to 1, the other to 1
    assert math.isclose(float(y[1]), -5.0 * sig(-1.702 * 5.0) * 0.0, abs_tol=1e-12)     # gate not cut below, the other to -1
    assert math.isclose(float(y[2]), 0.5 * sig(1.702 * 0.5) * 1.5)


def test_plain_router_weighs_the_chosen_logits_only():
    w = {"router": torch.eye(4, dtype=torch.float64), "router.b": torch.tensor([0.0, 0.0, 10.0, 0.0], dtype=torch.float64)}
    chosen, weights = plain.route(torch.tensor([[3.0, 1.0, -8.5, 1.5]], dtype=torch.float64), w, "", 2)     # logits 3, 1, 1.5, 1.5 + bias
    assert chosen.tolist() == [[0, 2]]                                      # the bias lifts expert 2 from last to second
    assert math.isclose(float(weights[0, 0]), math.exp(3.0) / (math.exp(3.0) + math.exp(1.5)))
    assert math.isclose(float(weights.sum()), 1.0)


# ----------------------------------------------------------------------------- kernels alone
import ctypes

from test_sopetar import _attend, _call, _meta, _pages, _rows_of     # launch helpers only (no test is imported)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,rows", [(48, 5), (36, 1), (64, 70), (6000, 3), (5, 9)])
def test_norm_behind_a_sub_layer_with_a_weight_stored_around_zero(dtype, width, rows):
    """h += rms(delta) * (1 + w), and the next reader's input is the stream itself in the activations' precision."""
    from mini_llm_runtime_b200.ops import native
    dev = "cuda:0"
    g = torch.Generator().manual_seed(width + rows)
    h, delta, w = torch.randn(rows, width, generator=g), 3.0 * torch.randn(rows, width, generator=g), 0.2 * torch.randn(width, generator=g).bfloat16().float()
    hd, dd = h.to(dev), delta.to(dev)
    weight = (w + 1.0).to(dev)
    out = torch.full((rows, width), float("nan"), dtype=dtype, device=dev)
    _call("norm_grouped", "mlr_group_rmsnorm", hd.data_ptr(), dd.data_ptr(), dd.stride(0), None, weight.data_ptr(), None, out.data_ptr(),
          out.stride(0), native.is_bf16(out), None, rows, width, 1, 1e-6, 3, native.stream())
    want = h.double() + plain.rms_norm(delta.double(), w.double(), 1e-6, one_plus=True)
    assert torch.allclose(hd.double().cpu(), want, atol=1e-5, rtol=1e-5)
    assert torch.equal(out.cpu(), hd.to(dtype).cpu())                     # the stream as it is, rounded once
    # the last norm of a model: wanted rows only, the stream unchanged
    rows_wanted = torch.tensor(sorted({0, rows - 1}), dtype=torch.int32, device=dev)
    before = hd.clone()
    last = torch.full((len(rows_wanted), width), float("nan"), dtype=dtype, device=dev)
    _call("norm_grouped", "mlr_group_rmsnorm", hd.data_ptr(), None, 0, None, None, weight.data_ptr(), last.data_ptr(), last.stride(0),
          native.is_bf16(last), rows_wanted.data_ptr(), len(rows_wanted), width, 1, 1e-6, 0, native.stream())
    want = plain.rms_norm(before.double().cpu()[rows_wanted.cpu().long()], w.double(), 1e-6, one_plus=True)
    tol = 1e-5 if dtype is torch.float32 else 2e-2
    assert torch.allclose(last.double().cpu(), want, atol=tol, rtol=tol) and torch.equal(hd, before)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,width,top,shared,gated", [(5, 48, 3, True, True), (70, 36, 1, False, False), (9, 256, 4, True, False), (300, 40, 2, True, True)])
def test_norm_behind_routed_experts_adds_up_their_pieces(rows, width, top, shared, gated):
    """The contribution given in pieces (a token's experts' results in rows ordered by expert, their weights, the shared expert's
    result and its gate): the launch adds them up, norms the sum and adds it into the stream."""
    from mini_llm_runtime_b200.ops import native
    dev = "cuda:0"
    g = torch.Generator().manual_seed(rows + width)
    h = torch.randn(rows, width, generator=g)
    y = torch.randn(rows * top, width, generator=g)
    row_of_pair = torch.randperm(rows * top, generator=g).to(torch.int32).view(rows, top)
    weights = torch.rand(rows, top, generator=g)
    other = torch.randn(rows, width, generator=g)
    gate = torch.rand(rows, generator=g)
    w = 0.2 * torch.randn(width, generator=g)
    hd, yd, rd, wd, od, gd, weight = (t.to(dev) for t in (h, y, row_of_pair, weights, other, gate, w + 1.0))
    out = torch.full((rows, width), float("nan"), dtype=torch.bfloat16, device=dev)
    _call("norm_grouped", "mlr_group_rmsnorm_pieces", hd.data_ptr(), yd.data_ptr(), width, rd.data_ptr(), wd.data_ptr(), top,
          od.data_ptr() if shared else None, od.stride(0) if shared else 0, gd.data_ptr() if shared and gated else None, weight.data_ptr(), None,
          out.data_ptr(), out.stride(0), 1, rows, width, 1, 1e-6, 3, native.stream())
    total = (weights.double()[:, :, None] * y.double()[row_of_pair.long()]).sum(dim=1)
    if shared:
        total = total + (gate.double()[:, None] if gated else 1.0) * other.double()
    want = h.double() + plain.rms_norm(total, w.double(), 1e-6, one_plus=True)
    assert torch.allclose(hd.double().cpu(), want, atol=2e-5, rtol=2e-5), float((hd.double().cpu() - want).abs().max())
    assert torch.equal(out.cpu(), hd.bfloat16().cpu())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width", [(3, 37), (70, 40), (2, 1024)])
def test_squared_relu_and_the_cap_on_the_logits(dtype, rows, width):
    from mini_llm_runtime_b200.ops import native
    dev = "cuda:0"
    g = torch.Generator().manual_seed(rows)
    x = (2.0 * torch.randn(rows, width, generator=g)).to(dtype).to(dev)
    want = torch.relu(x.double().cpu()) ** 2
    _call("elementwise", "mlr_activation", x.data_ptr(), x.stride(0), x.data_ptr(), x.stride(0), native.is_bf16(x), rows, width, 0, native.stream())
    tol = 1e-6 if dtype is torch.float32 else 1e-2
    assert torch.allclose(x.double().cpu(), want, atol=tol, rtol=tol)
    z = (20.0 * torch.randn(rows, width, generator=g)).to(dev)
    want = 7.5 * torch.tanh(z.double().cpu() / 7.5)
    _call("elementwise", "mlr_softcap", z.data_ptr(), rows, width, 7.5, native.stream())
    assert torch.allclose(z.double().cpu(), want, atol=2e-6, rtol=2e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,width,inter", [(1, 64, 48), (5, 256, 8192), (70, 40, 37), (1300, 256, 8192)])
def test_squared_relu_feed_forward_part_on_every_route(dtype, rows, width, inter):
    """The part by hand: few rows (the activation in the few-row product's epilogue), a portion (a kernel between the products)
    and a long portion of a wide layer (the activation in the epilogue of the two-SM tensor-core product)."""
    from mini_llm_runtime_b200.config.base import PartSpec
    from mini_llm_runtime_b200.csrc import build
    from mini_llm_runtime_b200.engine.runtime import Runtime
    from mini_llm_runtime_b200.parts.base import StepContext
    from mini_llm_runtime_b200.parts.mlp import PlainFeedForward
    g = torch.Generator().manual_seed(rows)
    w = {"up": (2.0 * torch.randn(inter, width, generator=g) / math.sqrt(width)).bfloat16(),
         "down": (torch.randn(width, inter, generator=g) / math.sqrt(inter)).bfloat16()}
    rt = Runtime(getattr(torch, dtype))
    part = PlainFeedForward(PartSpec("plain", {"hidden_size": width, "intermediate_size": inter, "activation": "relu2"}, {"up": "up", "down": "down"}))
    build.ensure(part.kernel_modules(rt.dtype) + ["host"])
    part.bind(w, rt)
    x = torch.randn(rows, width, generator=g).to(rt.dtype).to(rt.device)
    step = StepContext(rt=rt, num_rows=rows, segments=[], token_ids=None, positions=None, segment_of_row=None, segment_info=None, slots=None,
                       tables={}, page_size=16, status=torch.zeros(1, dtype=torch.int32, device=rt.device))
    got = part.forward(x, step).double().cpu()
    want = plain.squared_relu_ff(x.double().cpu(), {k: v.double() for k, v in w.items()}, "")
    tol = 1e-4 if dtype == "float32" else 3e-2
    assert torch.allclose(got, want, atol=tol * float(want.abs().max()), rtol=tol), float((got - want).abs().max())


def _mixer_case(kind, dtype, heads, kv_heads, dim, vdim, T, page, how="rows", window=None, rot=None, loud=None, scale=0.3, seed=0, reader=False):
    """The core of either mixer from given projections: `mlr_qkv_prepare_cache` (biases, the norm of q and k over the whole
    projection or per head, rotation of the keys, the cache) and then attention (window, sink and head gate, or causal with
    rotated queries), against the plain functions.  `loud`: a key position whose score with the last query stands far above
    all others on every head.  `reader`: the queries are prepared a second time by a launch without keys and values, as a
    layer does that reads another layer's cache; the cache must stay as it is."""
    from mini_llm_runtime_b200.ops import native
    from mini_llm_runtime_b200.ops.specs import GATES, QK_NORMS, MaskedAttentionSpec
    from mini_llm_runtime_b200.parts.rotary import scaled_frequencies
    import numpy as np
    dev = "cuda:0"
    windowed = kind == "attention"
    g = torch.Generator().manual_seed(seed + T)
    q, k, v = (torch.randn(T, n, generator=g) for n in (heads * dim, kv_heads * dim, kv_heads * vdim))
    bq, bk, bv = (torch.zeros(n) if windowed else 0.3 * torch.randn(n, generator=g) for n in (heads * dim, kv_heads * dim, kv_heads * vdim))
    wq = 1.0 + 0.2 * torch.randn(heads * dim if windowed else dim, generator=g)
    wk = 1.0 + 0.2 * torch.randn(kv_heads * dim if windowed else dim, generator=g)
    sink = 0.5 + torch.randn(heads, generator=g)
    gate = torch.randn(T, heads, generator=g)
    if loud is not None:
        # One column of every head carries the loud pair and is zero in every other key: the column after the rotated ones.
        col = dim - 1
        bq, bk = torch.zeros_like(bq), torch.zeros_like(bk)
        k.view(T, kv_heads, dim)[:, :, col] = 0.0
        k[loud] = 0.0
        k[loud].view(kv_heads, dim)[:, col] = 25.0
        q[T - 1] = 0.0
        q[T - 1].view(heads, dim)[:, col] = 25.0
        wq, wk = torch.ones_like(wq), torch.ones_like(wk)
    q, k, v, gate = (x.to(dtype).to(dev) for x in (q, k, v, gate))
    freqs, freq_dev = [], None
    if rot is not None:
        freqs = plain.scaled_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        mine = np.power(rot["base"], -2.0 * np.arange(rot["dims"] // 2) / rot["dims"])
        if rot.get("scaling"):
            mine = scaled_frequencies(mine, **rot["scaling"])
        freq_dev = torch.from_numpy(mine.astype(np.float32)).to(dev)
    keep = [t.float().to(dev) for t in (bq, bk, bv, wq, wk, sink)]
    spec = MaskedAttentionSpec(freq=freq_dev.data_ptr() if freq_dev is not None else None, sinks=keep[5].data_ptr() if windowed else None, slopes=None,
                               q_weight=keep[3].data_ptr(), k_weight=keep[4].data_ptr(), heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim,
                               rot_dims=rot["dims"] if rot else 0, window=window or 0, chunk=0, sink=int(windowed), gate_kind=GATES["sigmoid_head" if windowed else None],
                               shared_kv=0, keep_first=0, qk_norm=QK_NORMS["whole" if windowed else "head"], scale=scale, out_scale=1.0, softcap=0.0)
    cache, n_pages, table = _pages(T, page, kv_heads * (dim + vdim), dtype, g, dev)
    positions, of_row, _ = _meta([(0, T, 0, 0)], dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    raw_q = q.clone()
    biases = [None] * 3 if windowed else [t.data_ptr() for t in keep[:3]]
    _call("attention_masked", "mlr_qkv_prepare_cache", ctypes.addressof(spec), q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(),
          v.stride(0), native.is_bf16(q), *biases, 0, 0, 1e-5, None, 0, 0, 0.0, cache.data_ptr(), n_pages, positions.data_ptr(), of_row.data_ptr(),
          table.data_ptr(), table.stride(0), page, T, status.data_ptr(), native.stream())
    if reader:
        held, again = cache.clone(), raw_q.clone()
        _call("attention_masked", "mlr_qkv_prepare_cache", ctypes.addressof(spec), again.data_ptr(), again.stride(0), None, 0, None, 0, native.is_bf16(q),
              biases[0], None, None, 0, 0, 1e-5, None, 0, 0, 0.0, None, 0, positions.data_ptr(), of_row.data_ptr(), None, 0, page, T,
              status.data_ptr(), native.stream())
        assert torch.equal(again, q) and torch.equal(cache.view(torch.uint8), held.view(torch.uint8))
    assert int(status.item()) == 0
    out = torch.full((T, heads * vdim), float("nan"), dtype=dtype, device=dev)
    _attend(spec, q, gate if windowed else None, out, cache, n_pages, table, page, T, how, kv_heads, vdim)
    qd = raw_q.double().cpu() + bq.double()
    kd = k.double().cpu() + bk.double()
    vd = (v.double().cpu() + bv.double()).view(T, kv_heads, vdim)
    if windowed:
        qd = plain.rms_norm(qd, wq.double(), 1e-5).view(T, heads, dim)
        kd = plain.rms_norm(kd, wk.double(), 1e-5).view(T, kv_heads, dim)
        want = plain.attend(qd, kd, vd, scale, plain.visible(T, window), sink.double()) * torch.sigmoid(gate.double().cpu())[:, :, None]
    else:
        at = torch.arange(T)
        qd = plain.rotate_halves(plain.rms_norm(qd.view(T, heads, dim), wq.double(), 1e-5), at, freqs)
        kd = plain.rotate_halves(plain.rms_norm(kd.view(T, kv_heads, dim), wk.double(), 1e-5), at, freqs)
        want = plain.attend(qd, kd, vd, scale, plain.visible(T, None))
    rows = _rows_of(how, T)
    shown = torch.sigmoid(gate.double().cpu())[-1] if windowed else torch.ones(heads, dtype=torch.float64)
    return out.double().cpu()[rows], want.reshape(T, heads * vdim)[rows], vd, shown


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,rot_dims", [(4, 2, 64, 32), (2, 1, 128, 128), (3, 3, 16, 8), (2, 2, 40, 0)])
def test_preparation_for_the_plain_attention_kernels(dtype, heads, kv_heads, dim, rot_dims):
    """With `dense_cache` the launch rotates the queries in place and writes keys and values as the kernels of plain causal
    attention read them: [page][K | V][kv head][token][dim], the 16-byte chunks of a bfloat16 row of 64, 128 or 256 values
    exchanged by the position's last three bits."""
    from mini_llm_runtime_b200.ops import native
    from mini_llm_runtime_b200.ops.specs import MaskedAttentionSpec
    dev, T, page = "cuda:0", 37, 8
    g = torch.Generator().manual_seed(dim)
    q, k, v = (torch.randn(T, n, generator=g) for n in (heads * dim, kv_heads * dim, kv_heads * dim))
    bq, bk, bv = (0.3 * torch.randn(n, generator=g) for n in (heads * dim, kv_heads * dim, kv_heads * dim))
    wq, wk = 1.0 + 0.2 * torch.randn(dim, generator=g), 1.0 + 0.2 * torch.randn(dim, generator=g)
    freqs = plain.scaled_frequencies(300.0, rot_dims, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}) if rot_dims else []
    freq_dev = torch.tensor(freqs, dtype=torch.float32, device=dev) if rot_dims else None
    q, k, v = (x.to(dtype).to(dev) for x in (q, k, v))
    keep = [t.float().to(dev) for t in (bq, bk, bv, wq, wk)]
    spec = MaskedAttentionSpec(freq=freq_dev.data_ptr() if rot_dims else None, sinks=None, slopes=None, q_weight=keep[3].data_ptr(),
                               k_weight=keep[4].data_ptr(), heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, rot_dims=rot_dims, window=0, chunk=0,
                               sink=0, gate_kind=0, shared_kv=0, keep_first=0, qk_norm=1, dense_cache=1, scale=1.0, out_scale=1.0, softcap=0.0)
    cache, n_pages, table = _pages(T, page, 2 * kv_heads * dim, dtype, g, dev)
    positions, of_row, _ = _meta([(0, T, 0, 0)], dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    raw_q = q.clone()
    _call("attention_masked", "mlr_qkv_prepare_cache", ctypes.addressof(spec), q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(),
          v.stride(0), native.is_bf16(q), keep[0].data_ptr(), keep[1].data_ptr(), keep[2].data_ptr(), 0, 0, 1e-5, None, 0, 0, 0.0, cache.data_ptr(),
          n_pages, positions.data_ptr(), of_row.data_ptr(), table.data_ptr(), table.stride(0), page, T, status.data_ptr(), native.stream())
    assert int(status.item()) == 0
    at = torch.arange(T)
    want_q = plain.rotate_halves(plain.rms_norm((raw_q.double().cpu() + bq.double()).view(T, heads, dim), wq.double(), 1e-5), at, freqs)
    want_k = plain.rotate_halves(plain.rms_norm((k.double().cpu() + bk.double()).view(T, kv_heads, dim), wk.double(), 1e-5), at, freqs)
    want_v = (v.double().cpu() + bv.double()).view(T, kv_heads, dim)
    tol = 2e-5 if dtype is torch.float32 else 2e-2
    assert torch.allclose(q.double().cpu().view(T, heads, dim), want_q, atol=tol, rtol=tol)
    held = cache.double().cpu().view(n_pages, 2, kv_heads, page, dim)
    swizzled = dtype is torch.bfloat16 and dim in (64, 128, 256)
    for t in range(T):
        cols = torch.arange(dim)
        if swizzled:
            cols = cols ^ ((t & 7) << 3)
        where = held[int(table[0, t // page])][:, :, t % page][:, :, cols]          # [K | V][kv head][dim], columns put back
        assert torch.allclose(where[0], want_k[t], atol=tol, rtol=tol), t
        assert torch.allclose(where[1], want_v[t], atol=tol, rtol=tol), t


SCALED = {"base": 100.0, "dims": 8, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    dict(kind="attention", heads=4, kv_heads=2, dim=24, vdim=12, T=100, page=16, window=9),
    dict(kind="attention", heads=3, kv_heads=3, dim=10, vdim=6, T=70, page=4, window=1),
    dict(kind="attention", heads=2, kv_heads=1, dim=16, vdim=40, T=150, page=16, reader=True),
    dict(kind="attention", heads=4, kv_heads=1, dim=32, vdim=16, T=333, page=16, window=100, how=("split", 3, 64, 6, 1)),
    dict(kind="attention", heads=2, kv_heads=2, dim=16, vdim=24, T=700, page=8, window=200, how=("split", 1, 128, 6, 4)),
    dict(kind="attention_2", heads=4, kv_heads=2, dim=24, vdim=12, T=100, page=16, rot=SCALED, reader=True),
    dict(kind="attention_2", heads=5, kv_heads=5, dim=10, vdim=6, T=70, page=4, rot={"base": 50.0, "dims": 10}),
    dict(kind="attention_2", heads=2, kv_heads=1, dim=16, vdim=40, T=150, page=16),
    dict(kind="attention_2", heads=8, kv_heads=2, dim=32, vdim=16, T=333, page=16, rot={"base": 5e4, "dims": 16, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}},
         how=("split", 3, 64, 6, 1)),
    dict(kind="attention_2", heads=2, kv_heads=2, dim=16, vdim=24, T=700, page=8, rot=SCALED, how=("split", 1, 128, 6, 4)),
])
def test_both_mixers_from_given_projections(dtype, case):
    got, want, _, _ = _mixer_case(dtype=dtype, **case)
    tol = 3e-5 if dtype is torch.float32 else 3e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol), float((got - want).abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("case", [
    dict(kind="attention", heads=4, kv_heads=2, dim=32, vdim=16, T=200, page=16, window=40, how=("tiles", 70)),
    dict(kind="attention", heads=8, kv_heads=8, dim=16, vdim=8, T=333, page=4, window=100, how=("tiles", 1)),
    dict(kind="attention_2", heads=2, kv_heads=1, dim=96, vdim=96, T=150, page=16, rot={"base": 1e4, "dims": 48}, how=("tiles", 64)),
    dict(kind="attention_2", heads=4, kv_heads=2, dim=64, vdim=32, T=260, page=16, rot=SCALED, how=("tiles", 129)),
])
def test_the_same_in_tiles_on_the_tensor_cores(case):
    got, want, _, _ = _mixer_case(dtype=torch.bfloat16, **case)
    assert torch.allclose(got, want, atol=3e-2, rtol=3e-2), float((got - want).abs().max())


# (window, T, loud key, seen): the last query is at T - 1.
EDGES = [(50, 300, 250, True), (50, 300, 249, False), (64, 640, 576, True), (64, 640, 575, False), (1, 130, 129, True), (1, 130, 128, False),
         (None, 700, 0, True), (None, 700, 15, True), (None, 700, 16, True), (500, 700, 200, True), (500, 700, 199, False),
         (80, 200, 120, True), (80, 200, 119, False)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("how", ["rows", ("tiles", 130), ("split", 1, 64, 12, 1), ("split", 2, 128, 6, 4)])
def test_one_loud_key_just_inside_and_just_outside_the_window_and_far_back(dtype, how):
    """Among hundreds of keys one stands out for the last query.  If the mask lets the query see it (the window's oldest place, a
    key far back without a window, a page's last or first place) its value comes out, times the head's gate; one place further
    nothing of it does.  In a prompt's rows, in tiles, and as decoded tokens whose keys are cut into ranges; for the rotated
    mixer the far keys only (it has no window)."""
    if isinstance(how, tuple) and how[0] == "tiles" and dtype is not torch.bfloat16:
        pytest.skip("the tiled kernel is the bfloat16 one")
    tol = 3e-5 if dtype is torch.float32 else 3e-2
    for window, T, loud, seen in EDGES:
        for kind in ("attention", "attention_2"):
            if kind == "attention_2" and window is not None:
                continue
            got, want, values, shown = _mixer_case(kind, dtype, heads=2, kv_heads=1, dim=16, vdim=8, T=T, page=16, how=how, window=window,
                                                   rot=SCALED if kind == "attention_2" else None, loud=loud, scale=2.0)
            # The last row only: with a scale that makes one key loud, the other rows' scores are too large for what the
            # tolerance says of bfloat16 operands and of float32 angles at position 700 (the tests above compare whole prompts).
            assert torch.allclose(got[-1], want[-1], atol=tol, rtol=tol), (kind, window, T, loud, float((got[-1] - want[-1]).abs().max()))
            last, value = got[-1].view(2, 8), values[loud, 0].expand(2, 8) * shown[:, None]
            if seen:
                assert torch.allclose(last, value, atol=3e-2, rtol=3e-2), (kind, window, T, loud)
            else:
                assert float((last - value).abs().max()) > 0.1, (kind, window, T, loud)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows", [1, 3, 70, 300])
@pytest.mark.parametrize("experts,top,shared", [(6, 2, 20), (5, 5, 0), (7, 1, 9), (16, 4, 0)])
def test_routed_experts_with_clamped_gates_and_a_softmax_over_the_chosen(dtype, rows, experts, top, shared):
    """The part by hand against the plain functions: router logits with a bias, the chosen experts' weights, clamped experts,
    the shared expert behind its sigmoid gate."""
    from mini_llm_runtime_b200.config.base import PartSpec
    from mini_llm_runtime_b200.engine.runtime import Runtime
    from mini_llm_runtime_b200.parts.base import StepContext
    from mini_llm_runtime_b200.parts.experts import RoutedExperts
    width, inter = 40, 24
    g = torch.Generator().manual_seed(experts * 100 + rows)
    names = {"router": "router", "router_bias": "router.b"}
    w = {"router": (6.0 * torch.randn(experts, width, generator=g) / math.sqrt(width)).bfloat16(), "router.b": torch.randn(experts, generator=g).bfloat16()}
    made = [(f"e{i}.", inter) for i in range(experts)] + ([("shared.", shared)] if shared else [])
    for p, ff in made:
        for role, shape in (("gate", (ff, width)), ("up", (ff, width)), ("down", (width, ff))):
            names[p + role] = p + role
            w[p + role] = (2.0 * torch.randn(*shape, generator=g) / math.sqrt(shape[1])).bfloat16()
    if shared:
        names["shared.sg"] = "shared.sg"
        w["shared.sg"] = (2.0 * torch.randn(1, width, generator=g) / math.sqrt(width)).bfloat16()
    spec = PartSpec("routed_experts", {"hidden_size": width, "intermediate_size": inter, "experts": experts, "top": top, "router": "softmax_of_chosen",
                                       "activation": "swish", "alpha": 1.702, "up_offset": 1.0, "limit": 0.8, "shared_intermediate_size": shared or None,
                                       "shared_limit": 0.4 if shared else None}, names)
    rt = Runtime(getattr(torch, dtype))
    part = RoutedExperts(spec)
    from mini_llm_runtime_b200.csrc import build
    build.ensure(part.kernel_modules(rt.dtype))
    part.bind(w, rt)
    x = torch.randn(rows, width, generator=g).to(rt.dtype).to(rt.device)
    step = StepContext(rt=rt, num_rows=rows, segments=[], token_ids=None, positions=None, segment_of_row=None, segment_info=None, slots=None,
                       tables={}, page_size=16, status=torch.zeros(1, dtype=torch.int32, device=rt.device))
    got = part.forward(x, step).double().cpu()
    wide = {k: v.double() for k, v in w.items()}
    mlp = {"router": {"experts": experts, "top": top}, "expert": {"ff": inter, "limit": 0.8}}
    if shared:
        mlp["shared"] = {"ff": shared, "limit": 0.4}
    want = plain.routed_experts(x.double().cpu(), wide, "", mlp)
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol), float((got - want).abs().max())


# ----------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module", params=sorted(sokolorn_models.ALL))
def case(request, tmp_path_factory):
    config = sokolorn_models.get(request.param)
    weights = sokolorn_models.random_weights(config, seed=11)
    folder = str(tmp_path_factory.mktemp(request.param))
    write_model_folder(folder, config, weights)
    return folder, config, weights


CLOSE_CALL = 0.03       # a routing margin below this share of the largest logit can flip under bfloat16 rounding of the router's input


def settled_rows(config, weights, tokens):
    """Which positions choose their experts by a margin that bfloat16 rounding cannot overturn, in every layer."""
    margins = []
    plain.forward(config, {k: v.double() for k, v in weights.items()}, tokens, margins_out=margins)
    ok = torch.ones(len(tokens), dtype=torch.bool)
    for m in margins:
        ok &= m > CLOSE_CALL
    return ok


def close(got, want, dtype, what, settled=None):
    """float32: every row.  bfloat16: the rows whose choice of experts is no close call (a token that chooses another expert
    is another computation, not a rounding); they must be nearly all."""
    if dtype != "bfloat16":
        return assert_close(got, want, dtype, what)
    from helpers import assert_rows_close
    if settled is not None:
        assert int(settled.sum()) >= 0.5 * len(settled), f"{what}: too many close calls for a test ({int((~settled).sum())} of {len(settled)})"
        got, want = got[settled], want[settled]
    assert_rows_close(got, want, what, BF16)


@pytest.mark.gpu
def test_every_layer_of_a_short_prompt(case):
    """The stream after every layer, float32, with the steps driven from Python part by part."""
    from mini_llm_runtime_b200.engine.model import StepEntry
    folder, config, weights = case
    model = engine_model(folder, "float32", num_pages=8, page_size=8, max_requests=1)
    model._native = None
    seen = []
    for run in model.runs:
        def wrapped(h, pending, step, ctx, inner=run.block.forward):
            result = inner(h, pending, step, ctx)
            seen.append(h.double().cpu())
            return result
        run.block.forward = wrapped
    tokens = tokens_for(config, 19, 2)
    slot = model.open_request()
    model.step([StepEntry(slot, tokens, [18])])
    want = []
    plain.forward(config, {k: v.double() for k, v in weights.items()}, tokens, want)
    assert len(seen) == len(want)
    for i, (a, b) in enumerate(zip(seen, want)):
        assert torch.allclose(a, b, atol=2e-4, rtol=2e-4), (i, float((a - b).abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_portions_and_decoding_agree_with_the_plain_implementation(case, dtype):
    folder, config, weights = case
    model = engine_model(folder, dtype, num_pages=24, page_size=8, max_requests=2)
    assert model._native is not None, "the model must run in the native step executor"
    tokens = tokens_for(config, 150, 4)
    want = plain_logits(config, weights, tokens)
    settled = settled_rows(config, weights, tokens)
    whole = run_whole(model, tokens)
    close(whole, want, dtype, "whole", settled)
    for sizes in ([1], [2], [3, 2, 7], [64, 1], [65, 2, 70], [149, 1], [11, 2, 2, 30, 1, 5]):      # [1]: decoding from the first token on
        got = run_portions(model, tokens, sizes)
        close(got, want, dtype, f"portions {sizes}", settled)
        if dtype == "float32":      # how a prompt is cut changes nothing but the order of a few sums
            assert float((got - whole).abs().max()) <= 3e-5 * max(1.0, float(whole.abs().max())), sizes
    assert model.cache.free_slots() == 2


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_of_unequal_requests_equals_each_alone_and_slots_are_used_again(case, dtype):
    from mini_llm_runtime_b200.engine.model import StepEntry
    folder, config, weights = case
    model = engine_model(folder, dtype, num_pages=40, page_size=8, max_requests=3)
    lengths = [70, 9, 33, 2, 51, 20, 64]
    requests = [tokens_for(config, n, 100 + n) for n in lengths]
    alone = [plain_logits(config, weights, t) for t in requests]
    got = [[] for _ in requests]
    # Three live requests at a time; a finished one gives its slot and its pages to the next.
    waiting, live = list(range(len(requests))), {}
    sizes = [5, 1, 2, 13, 1, 1, 30, 3]
    turn = 0
    while waiting or live:
        while waiting and len(live) < 3:
            live[waiting.pop(0)] = [model.open_request(), 0]
        entries, who = [], []
        for i, (slot, at) in live.items():
            if (turn + i) % 4 == 3 and len(live) > 1:
                continue                                  # this request sits the step out
            n = min(sizes[(turn + i) % len(sizes)], len(requests[i]) - at)
            entries.append(StepEntry(slot, requests[i][at:at + n], list(range(n))))
            who.append((i, n))
        if entries:
            logits = model.step(entries).float().cpu()
            row = 0
            for i, n in who:
                got[i].append(logits[row:row + n])
                row += n
                live[i][1] += n
                if live[i][1] == len(requests[i]):
                    model.close_request(live.pop(i)[0])
        turn += 1
    model.check_status()
    for i in range(len(requests)):
        close(torch.cat(got[i]), alone[i], dtype, f"request {i}", settled_rows(config, weights, requests[i]) if len(requests[i]) > 9 else None)
    assert model.cache.free_slots() == 3


@pytest.mark.gpu
def test_long_decoding_through_the_graphs_passes_every_window(case):
    """Two requests decoded token by token from their first token on, far beyond every window of the small models, so that
    the caches with a window give pages back and take them again."""
    from mini_llm_runtime_b200.engine.model import StepEntry
    folder, config, weights = case
    model = engine_model(folder, "float32", num_pages=64, page_size=8, max_requests=2)
    a, b = tokens_for(config, 260, 1), tokens_for(config, 200, 2)
    sa, sb = model.open_request(), model.open_request()
    got_a, got_b = [], []
    for t in range(len(a)):
        entries = [StepEntry(sa, [a[t]], [0])] + ([StepEntry(sb, [b[t]], [0])] if t < len(b) else [])
        logits = model.step(entries).float().cpu()
        got_a.append(logits[0])
        if t < len(b):
            got_b.append(logits[1])
    model.check_status()
    assert model._graphs, "single-token steps did not reach the CUDA graphs"
    assert_close(torch.stack(got_a), plain_logits(config, weights, a), "float32", "a")
    assert_close(torch.stack(got_b), plain_logits(config, weights, b), "float32", "b")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(case, dtype):
    from mini_llm_runtime_b200 import LLM
    folder, config, weights = case
    prompts = [tokens_for(config, n, 50 + n) for n in (3, 41, 18, 77, 1)]
    llm = LLM(folder, dtype=dtype, max_model_len=128, max_requests=3, num_pages=48, page_size=8, max_batch_tokens=24, prefill_chunk=16)
    results = llm.generate(prompts, max_tokens=12, ignore_eos=True)
    for prompt, result in zip(prompts, results):
        assert len(result.token_ids) == 12
        tokens = list(prompt)
        for step, token in enumerate(result.token_ids):
            row = plain_logits(config, weights, tokens)[-1]
            best = int(torch.argmax(row))
            if token != best:       # two logits closer than the precision's rounding may change places; nothing else may
                margin = 1e-3 if dtype == "float32" else 2 * BF16["max"] * float(row.double().pow(2).mean().sqrt())
                assert float(row[best] - row[token]) <= margin, (len(prompt), step, token, best)
            tokens.append(token)
    assert llm.model.cache.free_slots() == 3


@pytest.mark.gpu
def test_trace_replay_with_a_pool_that_is_used_again(case, tmp_path):
    """Through `bin/trace_run` as a user runs it: up to four live requests in a pool sized for them, not for all."""
    import trace_tools
    folder, config, weights = case
    requests = {f"r{i}": tokens_for(config, n, 300 + i) for i, n in enumerate((90, 5, 130, 64, 31, 17, 100))}
    trace = trace_tools.mixed(requests, seed=9)
    logits = trace_tools.run_trace(folder, "float32", trace, str(tmp_path), config["vocab"])
    for name, tokens in requests.items():
        assert_close(trace_tools.stack(logits, name, len(tokens)), plain_logits(config, weights, tokens), "float32", name)
