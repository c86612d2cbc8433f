"""The Sopetar decoder: its mechanisms one by one against `plain_sopetar`, then whole models through the
engine's step function, scheduler and entry points.  The plain implementation shares nothing with the
package; it runs in float64 on bfloat16-rounded random weights."""
import ctypes
import math

import pytest
import torch

import plain_sopetar as plain
import sopetar_models
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
    for name in sopetar_models.ALL:
        config = sopetar_models.get(name)
        weights = sopetar_models.random_weights(config, 1)
        plan = plan_for(config_from_dict(config))
        expected = expected_weights(plan)
        assert set(expected) == set(weights), name
        for key, spec in expected.items():
            assert tuple(spec.shape) == tuple(weights[key].shape), key
        mixing = [layer.mixer.params.get("value_mix") for layer in plan.layers if layer.mixer.kind == "masked_attention"]
        mixing = [m for m in mixing if m is not None]
        assert mixing[:1] in ([], ["first"]) and all(m == "later" for m in mixing[1:]), name


@pytest.mark.parametrize("path,value,message", [
    (("width",), None, "width"),
    (("norm", "eps"), None, "eps"),
    (("layers", 0, "type"), "lightning", "latent_attention"),
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "mask", "keep_first"), -1, "keep_first"),
    (("layers", 1, "mixer", "rot"), None, "rot"),
    (("layers", 1, "mixer", "mask", "keep_first"), 2, "keep_first"),
    (("layers", 1, "mixer", "kv_rank"), None, "kv_rank"),
    (("layers", 2, "mixer", "vdim"), 16, "mix values"),
    (("layers", 0, "mlp", "kind"), "moe", "dense"),
    (("layers", 0, "mlp", "ff"), None, "ff"),
])
def test_config_errors_name_the_key(path, value, message):
    from mini_llm_runtime_b200 import models  # noqa: F401
    from mini_llm_runtime_b200.config.base import ConfigError
    from mini_llm_runtime_b200.config.registry import config_from_dict
    config = sopetar_models.get("small_a")
    at = config
    for key in path[:-1]:
        at = at[key]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        config_from_dict(config)


def test_plain_window_keeps_the_first_tokens_and_itself():
    seen = plain.visible(12, 4, 2)
    assert seen[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert seen[3].tolist() == [True] * 4 + [False] * 8
    assert plain.visible(5, 1)[4].tolist() == [False] * 4 + [True]
    assert plain.visible(5, None)[4].all()


def test_plain_sink_counts_once_and_has_no_value():
    scores = torch.tensor([[[0.0, 0.0]]], dtype=torch.float64)
    seen = torch.ones(1, 2, dtype=torch.bool)
    w = plain.softmax_with_sink(scores, seen, torch.tensor([math.log(2.0)], dtype=torch.float64))
    assert torch.allclose(w, torch.full((1, 1, 2), 0.25, dtype=torch.float64))
    w = plain.softmax_with_sink(scores, seen)
    assert torch.allclose(w, torch.full((1, 1, 2), 0.5, dtype=torch.float64))


def test_plain_rotation_turns_neighbouring_pairs_and_keeps_the_rest():
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0, 7.0]]], dtype=torch.float64)
    y = plain.rotate_pairs(x, torch.tensor([3]), 100.0, 4)
    a, b = 3.0, 3.0 * 100.0 ** (-0.5)
    want = [math.cos(a), math.sin(a), -2 * math.sin(b), 2 * math.cos(b), 5.0, 7.0]
    assert torch.allclose(y[0, 0], torch.tensor(want, dtype=torch.float64))
    # scores of rotated queries and keys depend on the distance only
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 8, generator=g, dtype=torch.float64), torch.randn(1, 1, 8, generator=g, dtype=torch.float64)
    s = [float((plain.rotate_pairs(q, torch.tensor([p + 5]), 50.0, 8) * plain.rotate_pairs(k, torch.tensor([p]), 50.0, 8)).sum()) for p in (0, 9, 400)]
    assert abs(s[0] - s[1]) < 1e-9 and abs(s[0] - s[2]) < 1e-9


def test_plain_feed_forward_clamps_the_gate_above_and_the_other_on_both_sides():
    w = {"gate": torch.eye(3, dtype=torch.float64), "up": torch.eye(3, dtype=torch.float64), "down": torch.eye(3, dtype=torch.float64),
         "gate.b": torch.zeros(3, dtype=torch.float64), "up.b": torch.zeros(3, dtype=torch.float64), "down.b": torch.zeros(3, dtype=torch.float64)}
    u = torch.tensor([[5.0, -5.0, 0.5]], dtype=torch.float64)
    y = plain.dense_feed_forward({"limit": 2.0}, w, "", u)[0]
    sw = lambda g: g / (1 + math.exp(-1.702 * g))
    assert torch.allclose(y, torch.tensor([sw(2.0) * 3.0, sw(-5.0) * -1.0, sw(0.5) * 1.5], dtype=torch.float64))
    y = plain.dense_feed_forward({}, w, "", u)[0]
    assert torch.allclose(y, torch.tensor([sw(5.0) * 6.0, sw(-5.0) * -4.0, sw(0.5) * 1.5], dtype=torch.float64))


def test_plain_distance_slopes_fall_by_halves_of_the_exponent():
    s = plain.distance_slopes(4)
    assert torch.allclose(s, torch.tensor([2.0 ** -2, 2.0 ** -4, 2.0 ** -6, 2.0 ** -8], dtype=torch.float64))


# ----------------------------------------------------------------------------- kernels alone
def _call(module, fn, *args):
    from mini_llm_runtime_b200.ops import native
    native.call(module, fn, *args)
    torch.cuda.synchronize()


def _meta(segments, device):
    """segments: (first row, count, start position, slot) -> positions, segment_of_row, segment_info on the device."""
    positions, of_row = [], []
    for i, (first, count, start, slot) in enumerate(segments):
        positions += list(range(start, start + count))
        of_row += [i] * count
    as_int = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    return as_int(positions), as_int(of_row), as_int(segments).reshape(-1, 4)


def _pages(T, page, width, dtype, g, dev, spare=3):
    """A cache of shuffled pages for one request of T tokens, filled with NaN: (cache, page count, table)."""
    n_pages = (T + page - 1) // page + spare
    order = torch.randperm(n_pages, generator=g)[:(T + page - 1) // page].to(torch.int32)
    return torch.full((n_pages, page * width), float("nan"), dtype=dtype, device=dev), n_pages, order.reshape(1, -1).to(dev)


def _attend(spec, q, gate, out, cache, n_pages, table, page, T, how, kv_heads, vdim):
    """The step's attention launches over rows 0..T-1 of one request whose keys lie in `cache`.  `how`: "rows" (one block a
    row and head), ("tiles", n) (bfloat16: tiles of 64 rows of two portions, the first of n rows), or ("split", rows, keys,
    most, finer) (the last rows as a segment of few rows whose keys are cut into ranges, as a step of decoded tokens runs)."""
    from mini_llm_runtime_b200.ops import native
    dev = q.device
    positions, of_row, _ = _meta([(0, T, 0, 0)], dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    common = (ctypes.addressof(spec), q.data_ptr(), q.stride(0), gate.data_ptr() if gate is not None else None,
              gate.stride(0) if gate is not None else 0, out.data_ptr(), out.stride(0))
    is16 = native.is_bf16(q)
    if how == "rows":
        _call("attention_masked", "mlr_attention_masked", *common, is16, cache.data_ptr(), n_pages, positions.data_ptr(), of_row.data_ptr(),
              table.data_ptr(), table.stride(0), page, T, None, 0, None, 0, 1, 1, None, status.data_ptr(), native.stream())
    elif how[0] == "tiles":
        first = how[1]
        info = torch.tensor([[0, first, 0, 0], [first, T - first, first, 0]], dtype=torch.int32, device=dev)
        tiles = torch.tensor([(0, t) for t in range(0, first, 64)] + [(1, t) for t in range(0, T - first, 64)], dtype=torch.int32, device=dev)
        two = torch.cat([table, table]).contiguous()
        _call("attention_masked", "mlr_attention_masked_tiles", *common, cache.data_ptr(), n_pages, tiles.data_ptr(), tiles.shape[0], info.data_ptr(),
              two.data_ptr(), two.stride(0), page, status.data_ptr(), native.stream())
    else:
        _, last, keys, most, finer = how
        info = torch.tensor([[T - last, last, T - last, 0]], dtype=torch.int32, device=dev)
        slots = max(16 * kv_heads, -(-spec.heads // 16) * 16)       # more than 16 heads on a kv head: one row, heads rounded up to 16
        partial = torch.full((slots * most * finer * (vdim + 2),), float("nan"), device=dev)
        _call("attention_masked", "mlr_attention_masked", *common, is16, cache.data_ptr(), n_pages, positions.data_ptr(), of_row.data_ptr(),
              table.data_ptr(), table.stride(0), page, 0, None, 1, info.data_ptr(), keys, most, finer, partial.data_ptr(), status.data_ptr(),
              native.stream())
    assert int(status.item()) == 0


def _rows_of(how, T):
    return slice(T - how[1], T) if isinstance(how, tuple) and how[0] == "split" else slice(0, T)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,states", [(48, 1), (36, 3), (64, 6), (6000, 2), (5, 9)])
def test_depth_average_and_layer_norm_kernel(dtype, width, states):
    """One launch: both sub-layers' results and a bias are added, the sum is stored as the newest state, the stream
    becomes the weighted sum of all states, and the layer norm of that is written out."""
    from mini_llm_runtime_b200.ops import native
    dev, rows = "cuda:0", 7
    g = torch.Generator().manual_seed(width + states)
    total = states + 2
    history = torch.randn(total, rows, width, generator=g).to(dev)
    h = torch.randn(rows, width, generator=g).to(dev)
    d1 = torch.randn(rows, width + 4, generator=g).to(dev)[:, :width]
    d2 = torch.randn(rows, width, generator=g).to(dev)
    bias, w, b = (torch.randn(width, generator=g).to(dev) for _ in range(3))
    dwa = torch.randn(states + 1, generator=g).to(dev)
    old_h, old_hist = h.clone(), history.clone()
    out = torch.full((rows, width), float("nan"), dtype=dtype, device=dev)
    _call("layernorm", "mlr_depth_norm", h.data_ptr(), d1.data_ptr(), d1.stride(0), d2.data_ptr(), d2.stride(0), bias.data_ptr(), history.data_ptr(),
          history.stride(0), states, dwa.data_ptr(), w.data_ptr(), b.data_ptr(), 1e-5, out.data_ptr(), out.stride(0), native.is_bf16(out), None, rows,
          width, 1, native.stream())
    newest = (old_h + d1 + d2 + bias).double().cpu()
    assert torch.allclose(history[states].double().cpu(), newest, atol=1e-5, rtol=1e-5)
    assert torch.equal(history[:states], old_hist[:states]) and torch.equal(history[states + 1:], old_hist[states + 1:])
    stream = plain.depth_average([old_hist[j].double().cpu() for j in range(states)] + [newest], dwa.double().cpu())
    assert torch.allclose(h.double().cpu(), stream, atol=1e-4, rtol=1e-5)
    want = plain.layer_norm(stream, w.double().cpu(), b.double().cpu(), 1e-5)
    tol = dict(atol=2e-4, rtol=2e-4) if dtype is torch.float32 else dict(atol=4e-2, rtol=2e-2)
    assert torch.allclose(out.double().cpu(), want, **tol)
    # the norm of chosen rows only (a model's last norm): nothing else changes
    chosen = torch.tensor([5, 0, 2], dtype=torch.int32, device=dev)
    before = h.clone()
    out2 = torch.full((3, width), float("nan"), dtype=dtype, device=dev)
    _call("layernorm", "mlr_depth_norm", h.data_ptr(), None, 0, None, 0, None, None, 0, 0, None, w.data_ptr(), b.data_ptr(), 1e-3, out2.data_ptr(),
          out2.stride(0), native.is_bf16(out2), chosen.data_ptr(), 3, width, 0, native.stream())
    want2 = plain.layer_norm(stream[[5, 0, 2]], w.double().cpu(), b.double().cpu(), 1e-3)
    assert torch.allclose(out2.double().cpu(), want2, **tol) and torch.equal(before, h)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter,limit,alpha,offset", [(37, 0.5, 1.702, 1.0), (40, 3.0, 1.0, 0.0), (1024, 0.0, 1.702, 1.0), (8, 1.0, 0.5, -2.0)])
def test_clamped_gate_kernel(dtype, inter, limit, alpha, offset):
    from mini_llm_runtime_b200.ops import native
    dev, rows = "cuda:0", 6
    g = torch.Generator().manual_seed(inter)
    both = (2.0 * torch.randn(rows, 2 * inter, generator=g)).to(dtype).to(dev)
    bg, bu = torch.randn(inter, generator=g).to(dev), torch.randn(inter, generator=g).to(dev)
    out = torch.full((rows, inter), float("nan"), dtype=dtype, device=dev)
    _call("elementwise", "mlr_gated_bias_shaped", both.data_ptr(), 2 * inter, bg.data_ptr(), bu.data_ptr(), out.data_ptr(), inter, native.is_bf16(out),
          rows, inter, 2, alpha, limit, offset, native.stream())
    z = both[:, :inter].double().cpu() + bg.double().cpu()
    up = both[:, inter:].double().cpu() + bu.double().cpu()
    if limit:
        z, up = torch.clamp(z, max=limit), torch.clamp(up, -limit, limit)
    want = z * torch.sigmoid(alpha * z) * (up + offset)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype is torch.float32 else dict(atol=2e-2, rtol=1e-2)
    assert torch.allclose(out.double().cpu(), want, **tol)


def _biased_attention_case(dtype, heads, kv_heads, dim, vdim, T, page, how="rows", window=None, keep_first=0, softcap=None, unit=True,
                           bias=True, mix=None, loud=None, scale=0.3, seed=0):
    """`mlr_qkv_prepare_cache` (biases, unit heads, mixed values, the cache) and then attention with the capped score, the
    distance bias and the window that keeps first tokens, against the plain functions.  `mix`: None, "first" or a lambda.
    `loud`: a key position whose score with the last query is made to stand far above all others (on every head)."""
    from mini_llm_runtime_b200.ops import native
    from mini_llm_runtime_b200.ops.specs import GATES, MaskedAttentionSpec
    dev = "cuda:0"
    g = torch.Generator().manual_seed(seed + T)
    q, k, v = (torch.randn(T, n, generator=g) for n in (heads * dim, kv_heads * dim, kv_heads * vdim))
    bq, bk, bv = (0.3 * torch.randn(n, generator=g) if bias else torch.zeros(n) for n in (heads * dim, kv_heads * dim, kv_heads * vdim))
    if loud is not None:
        assert not unit and not bias
        k[loud] = 0.0
        k[loud].view(kv_heads, dim)[:, 0] = 25.0
        q[T - 1] = 0.0
        q[T - 1].view(heads, dim)[:, 0] = 25.0
    v_first = torch.randn(T, kv_heads * vdim, generator=g)
    q, k, v = (x.to(dtype).to(dev) for x in (q, k, v))
    slopes = plain.distance_slopes(heads)
    slopes_dev = slopes.float().to(dev)
    spec = MaskedAttentionSpec(freq=None, sinks=None, slopes=slopes_dev.data_ptr(), heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot_dims=0,
                               window=window or 0, chunk=0, sink=0, gate_kind=GATES[None], shared_kv=0, keep_first=keep_first if window else 0,
                               scale=scale, out_scale=1.0, softcap=softcap or 0.0)
    cache, n_pages, table = _pages(T, page, kv_heads * (dim + vdim), dtype, g, dev)
    positions, of_row, _ = _meta([(0, T, 0, 0)], dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    first = v_first.clone().to(dev) if mix is not None else None
    dev_or_none = lambda t: t.to(dev).data_ptr() if bias else None
    keep = [bq.to(dev), bk.to(dev), bv.to(dev)]
    raw_q = q.clone()
    _call("attention_masked", "mlr_qkv_prepare_cache", ctypes.addressof(spec), q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(),
          v.stride(0), native.is_bf16(q), keep[0].data_ptr() if bias else None, keep[1].data_ptr() if bias else None,
          keep[2].data_ptr() if bias else None, int(unit), int(unit), 1e-5, first.data_ptr() if first is not None else None,
          first.stride(0) if first is not None else 0, 0 if mix is None else (1 if mix == "first" else 2), 0.0 if mix in (None, "first") else mix,
          cache.data_ptr(), n_pages, positions.data_ptr(), of_row.data_ptr(), table.data_ptr(), table.stride(0), page, T, status.data_ptr(),
          native.stream())
    assert int(status.item()) == 0
    out = torch.full((T, heads * vdim), float("nan"), dtype=dtype, device=dev)
    _attend(spec, q, None, out, cache, n_pages, table, page, T, how, kv_heads, vdim)
    qd = raw_q.double().cpu().view(T, heads, dim) + bq.double().view(heads, dim)
    kd = k.double().cpu().view(T, kv_heads, dim) + bk.double().view(kv_heads, dim)
    vd = v.double().cpu().view(T, kv_heads, vdim) + bv.double().view(kv_heads, vdim)
    if unit:
        qd, kd, vd = plain.unit_rms(qd, 1e-5), plain.unit_rms(kd, 1e-5), plain.unit_rms(vd, 1e-5)
    if mix == "first":
        assert torch.allclose(first.double().cpu().view(T, kv_heads, vdim), vd, atol=1e-5 if dtype is torch.float32 else 2e-2, rtol=1e-2)
    elif mix is not None:
        vd = (1.0 - mix) * vd + mix * v_first.double().view(T, kv_heads, vdim)
    rep = heads // kv_heads
    want = plain.attend(qd, kd.repeat_interleave(rep, dim=1), vd.repeat_interleave(rep, dim=1), scale, plain.visible(T, window, keep_first),
                        softcap, slopes)
    rows = _rows_of(how, T)
    return out.double().cpu()[rows], want.reshape(T, heads * vdim)[rows], vd


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    dict(heads=4, kv_heads=2, dim=24, vdim=12, T=100, page=16, window=9, keep_first=3, softcap=4.0, mix="first"),
    dict(heads=3, kv_heads=3, dim=10, vdim=6, T=70, page=4, window=3, keep_first=8, softcap=2.0, mix=0.35),
    dict(heads=2, kv_heads=1, dim=16, vdim=40, T=150, page=16, bias=False),
    dict(heads=6, kv_heads=2, dim=8, vdim=8, T=90, page=8, window=1, keep_first=2, unit=False, scale=0.1, mix=0.8),
    dict(heads=1, kv_heads=1, dim=130, vdim=200, T=200, page=16, window=64, softcap=30.0),
    dict(heads=4, kv_heads=1, dim=32, vdim=16, T=333, page=16, window=100, keep_first=70, softcap=10.0, how=("split", 3, 64, 6, 1)),
    dict(heads=2, kv_heads=2, dim=16, vdim=24, T=700, page=8, window=200, keep_first=5, how=("split", 1, 128, 6, 4), mix="first"),
])
def test_attention_with_biases_unit_heads_cap_distance_bias_and_kept_first_tokens(dtype, case):
    got, want, _ = _biased_attention_case(dtype, **case)
    tol = 3e-5 if dtype is torch.float32 else 3e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol), float((got - want).abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("case", [
    dict(heads=4, kv_heads=2, dim=32, vdim=16, T=200, page=16, window=40, keep_first=70, softcap=10.0, how=("tiles", 70)),
    dict(heads=8, kv_heads=8, dim=16, vdim=8, T=333, page=4, window=100, keep_first=1, how=("tiles", 1), mix=0.5),
    dict(heads=2, kv_heads=1, dim=96, vdim=96, T=150, page=16, softcap=50.0, how=("tiles", 64)),
    dict(heads=2, kv_heads=2, dim=64, vdim=32, T=260, page=16, window=80, keep_first=5, softcap=20.0, how=("tiles", 129), mix="first"),
])
def test_the_same_in_tiles_on_the_tensor_cores(case):
    got, want, _ = _biased_attention_case(torch.bfloat16, **case)
    assert torch.allclose(got, want, atol=3e-2, rtol=3e-2), float((got - want).abs().max())


# (window, kept first tokens, T, loud key, seen): the last query is at T - 1.
EDGES = [(50, 4, 300, 250, True), (50, 4, 300, 249, False), (50, 4, 300, 3, True), (50, 4, 300, 4, False), (50, 0, 300, 0, False),
         (64, 1, 640, 576, True), (64, 1, 640, 575, False), (64, 1, 640, 0, True), (64, 1, 640, 1, False),
         (1, 0, 130, 129, True), (1, 0, 130, 128, False), (None, 0, 700, 0, True), (None, 0, 700, 15, True), (None, 0, 700, 16, True),
         (500, 0, 700, 200, True), (500, 0, 700, 199, False), (7, 70, 400, 69, True), (7, 70, 400, 70, False), (7, 70, 400, 393, True)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("how", ["rows", ("tiles", 130), ("split", 1, 64, 12, 1), ("split", 2, 128, 6, 4)])
def test_one_loud_key_just_inside_and_just_outside_the_window_and_the_kept_tokens(dtype, how):
    """Among hundreds of keys one stands out for the last query.  If the mask lets the query see it (the window's oldest
    place, the last kept token, a key far back without a window, a page's last or first place) its value comes out; if it
    lies one place further (the first outside the window, the first that is not kept) nothing of it does.  In a prompt's
    rows, in tiles, and as decoded tokens whose keys are cut into ranges."""
    if isinstance(how, tuple) and how[0] == "tiles" and dtype is not torch.bfloat16:
        pytest.skip("the tiled kernel is the bfloat16 one")
    for window, keep, T, loud, seen in EDGES:
        got, want, values = _biased_attention_case(dtype, heads=2, kv_heads=1, dim=16, vdim=8, T=T, page=16, how=how, window=window, keep_first=keep,
                                                   softcap=900.0, unit=False, bias=False, loud=loud, scale=0.5)
        tol = 3e-5 if dtype is torch.float32 else 3e-2
        assert torch.allclose(got, want, atol=tol, rtol=tol), (window, keep, T, loud, float((got - want).abs().max()))
        last, value = got[-1].view(2, 8), values[loud, 0].expand(2, 8)
        if seen:
            assert torch.allclose(last, value, atol=3e-2, rtol=3e-2), (window, keep, T, loud)
        else:
            assert float((last - value).abs().max()) > 0.2, (window, keep, T, loud)


def _latent_case(dtype, heads, dim, rot, vdim, rank, T, page, how="rows", window=None, base=10000.0, loud=None, seed=0):
    """The kernels of a latent mixer between its first and its last product: the latent's norm, the rotation of the shared
    key part and of the queries' rotated parts, the cache, the queries through their heads' key matrices, attention over the
    cached vectors with a learned sink and a gate per head, and the result through the heads' value matrices; against
    `plain.latent_attention` with the two outer products done here.  `loud`: a position whose latent is made to stand out
    for the last query."""
    from mini_llm_runtime_b200.ops import native
    from mini_llm_runtime_b200.ops.specs import GATES, MaskedAttentionSpec
    dev, W = "cuda:0", 24
    g = torch.Generator().manual_seed(seed + T + rank)
    w = {"q": torch.randn(heads * (dim + rot), W, generator=g) / math.sqrt(W), "dkv": torch.randn(rank + rot, W, generator=g) / math.sqrt(W),
         "dkv.norm": 1.0 + 0.2 * torch.randn(rank, generator=g), "uk": torch.randn(heads * dim, rank, generator=g) / math.sqrt(rank),
         "uv": torch.randn(heads * vdim, rank, generator=g) / math.sqrt(rank), "sink": torch.randn(heads, generator=g),
         "g": torch.randn(heads, W, generator=g) / math.sqrt(W), "o": torch.eye(heads * vdim)}
    w = {k: v.to(dtype).double() for k, v in w.items()}
    u = torch.randn(T, W, generator=g).to(dtype).double()
    scale = 0.4
    if loud is not None:
        # Two inputs are markers: the first is set for the loud token only and is all that row 1 of the down projection reads, so
        # that the loud token's latent is one large value at place 1 and no other latent has anything there; the second is set
        # for the last token only and is all that the queries read.  Every head's key matrix maps the first query value to place 1.
        u[:, :2] = 0.0
        u[loud, 0] = 1.0
        u[T - 1, 1] = 1.0
        w["dkv"][:, 0] = 0.0
        w["dkv"][1] = 0.0
        w["dkv"][1, 0] = 50.0
        uk = w["uk"].view(heads, dim, rank)
        uk[:, 0] = 0.0
        uk[:, 0, 1] = 1.0
        qw = w["q"].view(heads, dim + rot, W)
        qw[:] = 0.0
        qw[:, 0, 1] = 30.0
    proj = torch.cat([u @ w["q"].T, u @ w["dkv"].T, u @ w["g"].T], dim=1).to(dtype).to(dev).contiguous()
    down_at, gate_at, key = heads * (dim + rot), heads * (dim + rot) + rank + rot, rank + rot
    norm_w = w["dkv.norm"].float().to(dev)
    sinks = w["sink"].float().to(dev)
    freq = torch.tensor([base ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)], dtype=torch.float32, device=dev)
    cache, n_pages, table = _pages(T, page, key, dtype, g, dev)
    positions, of_row, _ = _meta([(0, T, 0, 0)], dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    q = torch.full((T, heads * key), float("nan"), dtype=dtype, device=dev)
    down = proj[:, down_at:]
    is16 = native.is_bf16(proj)
    _call("latent", "mlr_latent_rot_cache", down.data_ptr(), down.stride(0), is16, norm_w.data_ptr(), 1e-5, rank, rot, rot, 1,
          freq.data_ptr() if rot else None, proj.data_ptr(), proj.stride(0), dim, dim + rot, heads, q.data_ptr(), q.stride(0), rank, key, cache.data_ptr(),
          n_pages, positions.data_ptr(), of_row.data_ptr(), table.data_ptr(), table.stride(0), page, 1, T, status.data_ptr(), native.stream())
    w_uk = w["uk"].view(heads, dim, rank).to(dtype).to(dev).contiguous()
    w_uv = w["uv"].view(heads, vdim, rank).transpose(1, 2).to(dtype).to(dev).contiguous()
    _call("latent", "mlr_head_project_strided", proj.data_ptr(), proj.stride(0), dim + rot, w_uk.data_ptr(), q.data_ptr(), q.stride(0), key, is16, T,
          heads, dim, rank, native.stream())
    assert not torch.isnan(q.float()).any()
    spec = MaskedAttentionSpec(freq=None, sinks=sinks.data_ptr(), slopes=None, heads=heads, kv_heads=1, dim=key, vdim=rank, rot_dims=0,
                               window=window or 0, chunk=0, sink=1, gate_kind=GATES["sigmoid_head"], shared_kv=1, keep_first=0, scale=scale,
                               out_scale=1.0, softcap=0.0)
    mixed = torch.full((T, heads * rank), float("nan"), dtype=dtype, device=dev)
    gate = proj[:, gate_at:]
    _attend(spec, q, gate, mixed, cache, n_pages, table, page, T, how, 1, rank)
    rows = _rows_of(how, T)
    mixed[:rows.start] = 0.0        # rows that this way of running does not compute
    act = torch.full((T, heads * vdim), float("nan"), dtype=dtype, device=dev)
    _call("latent", "mlr_head_project_strided", mixed.data_ptr(), mixed.stride(0), rank, w_uv.data_ptr(), act.data_ptr(), act.stride(0), vdim, is16, T,
          heads, rank, vdim, native.stream())
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": {"base": base, "dims": rot}}
    if window:
        m["mask"] = {"size": window}
    want = plain.latent_attention(m, w, "", u, 1e-5)
    latents = plain.unit_rms((u @ w["dkv"].T)[:, :rank], 1e-5) * w["dkv.norm"]
    return act.double().cpu()[rows], want[rows], latents, w, u


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    dict(heads=3, dim=8, rot=4, vdim=12, rank=16, T=100, page=16, window=7),
    dict(heads=5, dim=10, rot=6, vdim=6, rank=12, T=70, page=4, window=1, base=100.0),
    dict(heads=2, dim=16, rot=8, vdim=8, rank=24, T=150, page=8),
    dict(heads=1, dim=12, rot=2, vdim=20, rank=12, T=90, page=16, window=33, base=50.0),
    dict(heads=4, dim=16, rot=16, vdim=8, rank=48, T=333, page=16, window=70, how=("split", 3, 64, 6, 1)),
    dict(heads=2, dim=32, rot=32, vdim=16, rank=32, T=700, page=16, window=300, how=("split", 1, 128, 6, 4), base=500.0),
    dict(heads=2, dim=8, rot=0, vdim=8, rank=16, T=60, page=16, window=20),
    # more than 16 heads on the one kv head: a decoded token's heads are taken 16 at a time, with and without ranges of keys
    dict(heads=20, dim=16, rot=16, vdim=8, rank=48, T=333, page=16, window=70, how=("split", 1, 64, 6, 1)),
    dict(heads=35, dim=8, rot=8, vdim=8, rank=24, T=210, page=8, how=("split", 1, 64, 1, 1)),
    dict(heads=33, dim=16, rot=16, vdim=8, rank=32, T=500, page=16, window=260, how=("split", 1, 128, 3, 4), base=500.0),
])
def test_latent_attention_with_a_rotated_key_part_a_window_a_sink_and_a_gate(dtype, case):
    got, want, *_ = _latent_case(dtype, **case)
    tol = 5e-5 if dtype is torch.float32 else 4e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol), float((got - want).abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("case", [
    dict(heads=4, dim=16, rot=16, vdim=8, rank=48, T=200, page=16, window=70, how=("tiles", 70)),
    dict(heads=2, dim=32, rot=32, vdim=16, rank=32, T=333, page=4, how=("tiles", 1), base=500.0),
    dict(heads=3, dim=48, rot=16, vdim=24, rank=80, T=260, page=16, window=90, how=("tiles", 129)),
])
def test_the_latent_mixer_in_tiles_on_the_tensor_cores(case):
    got, want, *_ = _latent_case(torch.bfloat16, **case)
    assert torch.allclose(got, want, atol=4e-2, rtol=4e-2), float((got - want).abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("how", ["rows", ("tiles", 130), ("split", 1, 64, 12, 1), ("split", 2, 128, 6, 4)])
def test_one_loud_latent_just_inside_and_just_outside_the_window(dtype, how):
    """The same for the latent mixer: the last query's weight goes to one chosen token's latent if the window holds it, and
    the head's result is then that latent through the head's value matrix (times the gate)."""
    if isinstance(how, tuple) and how[0] == "tiles" and dtype is not torch.bfloat16:
        pytest.skip("the tiled kernel is the bfloat16 one")
    for window, T, loud, seen in [(50, 300, 250, True), (50, 300, 249, False), (64, 640, 576, True), (64, 640, 575, False), (1, 130, 129, True),
                                  (1, 130, 128, False), (None, 700, 0, True), (None, 700, 15, True), (None, 700, 16, True), (500, 700, 200, True),
                                  (500, 700, 199, False)]:
        got, want, latents, w, u = _latent_case(dtype, heads=2, dim=16, rot=16, vdim=8, rank=32, T=T, page=16, how=how, window=window, loud=loud)
        tol = 5e-5 if dtype is torch.float32 else 4e-2
        assert torch.allclose(got, want, atol=tol, rtol=tol), (window, T, loud, float((got - want).abs().max()))
        value = (latents[loud] @ w["uv"].T).view(2, 8) * torch.sigmoid(u[T - 1] @ w["g"].T)[:, None]
        last = got[-1].view(2, 8)
        if seen:
            assert torch.allclose(last, value, atol=4e-2, rtol=4e-2), (window, T, loud)
        else:
            assert float((last - value).abs().max()) > 0.05, (window, T, loud)


# ----------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module", params=sorted(sopetar_models.ALL))
def case(request, tmp_path_factory):
    config = sopetar_models.get(request.param)
    weights = sopetar_models.random_weights(config, seed=11)
    folder = str(tmp_path_factory.mktemp(request.param))
    write_model_folder(folder, config, weights)
    return folder, config, weights


def close(got, want, dtype, what):
    if dtype != "bfloat16":
        return assert_close(got, want, dtype, what)
    from helpers import assert_rows_close
    assert_rows_close(got, want, what, BF16)


@pytest.mark.gpu
def test_every_layer_of_a_short_prompt(case):
    """The stream after every layer (after its average over depth), float32, with the steps driven from Python part by part."""
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
    whole = run_whole(model, tokens)
    close(whole, want, dtype, "whole")
    for sizes in ([1], [2], [3, 2, 7], [64, 1], [65, 2, 70], [149, 1], [11, 2, 2, 30, 1, 5]):      # [1]: decoding from the first token on
        got = run_portions(model, tokens, sizes)
        close(got, want, dtype, f"portions {sizes}")
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
        close(torch.cat(got[i]), alone[i], dtype, f"request {i}")
    assert model.cache.free_slots() == 3


@pytest.mark.gpu
def test_long_decoding_through_the_graphs_passes_every_window(case):
    """Two requests decoded token by token from their first token on, far beyond every window of the small models, so that
    the caches with a window give pages back and take them again while the kept first tokens stay."""
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
