"""The Niridra decoder: its mechanisms one by one against `plain_niridra`, then whole models through the
engine's step function, scheduler and entry points.  The plain implementation shares nothing with the
package; it runs in float64 on bfloat16-rounded random weights."""
import ctypes
import math
import os

import pytest
import torch

import niridra_models
import plain_niridra as plain
from helpers import assert_close, engine_model, run_portions, run_whole, write_model_folder

# bfloat16 rows against the float64 plain implementation (relative RMSE, relative largest difference, cosine): a factor
# of two above the worst rows these narrow models measure.  A wrong key, a lost state, a wrong expert or a wrong pair row
# moves a row by its whole size; the float32 runs of the same tests are the sharp ones.
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
    for name in niridra_models.ALL:
        config = niridra_models.get(name)
        weights = niridra_models.random_weights(config, 1)
        plan = plan_for(config_from_dict(config))
        expected = expected_weights(plan)
        assert set(expected) == set(weights), name
        for key, spec in expected.items():
            assert tuple(spec.shape) == tuple(weights[key].shape), key
        for i, layer in enumerate(config["layers"]):
            assert plan.schedule[i].kv_from == layer["mixer"].get("kv_from")


@pytest.mark.parametrize("path,value,message", [
    (("width",), None, "width"),
    (("embedding", "scale"), None, "scale"),
    (("embedding", "bigram", "buckets"), 0, "buckets"),
    (("layers", 0, "type"), "delta", "lightning"),
    (("layers", 1, "mixer", "decay"), [0.5], "decay"),
    (("layers", 2, "mixer", "kv_from"), 1, "kv_from"),
    (("layers", 2, "mixer", "kv_from"), 2, "earlier"),
    (("layers", 2, "mixer", "kv_rank"), 32, "kv_from"),
    (("layers", 0, "mlp", "kind"), "dense", "moe"),
    (("layers", 0, "mlp", "router", "top"), 5, "cannot give"),
    (("layers", 3, "mlp", "router", "groups", "count"), 3, "cannot give"),
])
def test_config_errors_name_the_key(path, value, message):
    from mini_llm_runtime_b200 import models  # noqa: F401
    from mini_llm_runtime_b200.config.base import ConfigError
    from mini_llm_runtime_b200.config.registry import config_from_dict
    config = niridra_models.get("small_a")
    at = config
    for key in path[:-1]:
        at = at[key]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        config_from_dict(config)


def test_plain_lightning_attention_is_the_decayed_sum_of_outer_products():
    g = torch.Generator().manual_seed(5)
    T, H, D, Dv = 9, 2, 4, 3
    q, k, v = (torch.randn(T, H, n, generator=g, dtype=torch.float64) for n in (D, D, Dv))
    decay = [0.5, 1.0]
    out = plain.lightning_attention(q, k, v, decay)
    for h in range(H):
        for t in range(T):
            want = sum(decay[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
            assert torch.allclose(out[t, h], want, atol=1e-12)


def test_plain_router_keeps_to_the_best_groups_also_below_zero():
    # Every choice is negative; group 1 holds the two largest of all, group 0 the third: with one kept group and two
    # chosen experts both come from group 1, and the weights are the plain scores over their sum.
    z = torch.tensor([[-1.0, -9.0, -0.2, -0.5]], dtype=torch.float64)
    correction = torch.full((4,), -2.0, dtype=torch.float64)
    chosen, weights = plain.route(z, torch.eye(4, dtype=torch.float64), correction, 2, 2, 1)
    assert sorted(chosen[0].tolist()) == [2, 3]
    s = torch.sigmoid(z[0])
    assert torch.allclose(weights[0].sum(), torch.tensor(1.0, dtype=torch.float64))
    assert torch.allclose(weights[0, 0] / weights[0, 1], s[chosen[0, 0]] / s[chosen[0, 1]])


def test_plain_pair_rows():
    assert plain.bigram_rows([5, 2, 9], 7, 3, 4) == [7, (5 * 3 + 2 * 4) % 7, (2 * 3 + 9 * 4) % 7]


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


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams,buckets", [(1, 0), (3, 11), (8, 1)])
def test_hashed_embedding_kernel_over_steps(dtype, streams, buckets):
    """Two requests in slots 2 and 0, three steps each cut differently; a slot used again starts from the extra row."""
    from mini_llm_runtime_b200.ops import native
    dev, V, W = "cuda:0", 23, 20
    g = torch.Generator().manual_seed(1)
    table = torch.randn(V, W, generator=g).to(dtype).to(dev)
    pairs = torch.randn(buckets + 1, W, generator=g).to(dtype).to(dev) if buckets else None
    state = torch.full((3, 1), 77, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    seqs = {2: torch.randint(0, V, (9,), generator=g).tolist(), 0: torch.randint(0, V, (6,), generator=g).tolist()}
    cuts = {2: [4, 1, 4], 0: [1, 2, 3]}
    got = {2: [], 0: []}
    at = {2: 0, 0: 0}
    for step in range(3):
        segments, ids, row = [], [], 0
        for slot in (2, 0):
            n = cuts[slot][step]
            segments.append((row, n, at[slot], slot))
            ids += seqs[slot][at[slot]:at[slot] + n]
            row += n
        _, of_row, info = _meta(segments, dev)
        ids_t = torch.tensor(ids, dtype=torch.int32, device=dev)
        h = torch.full((row, streams * W), float("nan"), device=dev)
        _call("streams", "mlr_embed_hashed", h.data_ptr(), table.data_ptr(), pairs.data_ptr() if buckets else None, native.is_bf16(table),
              ids_t.data_ptr(), of_row.data_ptr(), info.data_ptr(), state.data_ptr(), state.stride(0), row, W, V, streams, 1.75, buckets, 5, 3,
              status.data_ptr(), native.stream())
        for first, n, start, slot in segments:
            got[slot].append(h[first:first + n].cpu())
            at[slot] += n
    assert int(status.item()) == 0
    for slot, seq in seqs.items():
        want = plain.embed(seq, table.double().cpu(), 1.75, pairs.double().cpu() if buckets else None, buckets, 5, 3)
        have = torch.cat(got[slot]).double().view(len(seq), streams, W)
        for s in range(streams):
            assert torch.allclose(have[:, s], want, atol=1e-5, rtol=1e-6), (slot, s)
    if buckets:
        assert state[:, 0].tolist() == [seqs[0][-1], 77, seqs[2][-1]]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams,width", [(1, 40), (4, 48), (8, 6), (3, 13000)])
def test_streams_step_kernel(dtype, streams, width):
    from mini_llm_runtime_b200.ops import native
    dev, rows = "cuda:0", 5
    g = torch.Generator().manual_seed(streams)
    h = torch.randn(rows, streams * width, generator=g).to(dev)
    y = torch.randn(rows, width + 3, generator=g).to(dev)[:, :width]
    scale, norm_w = torch.randn(width, generator=g).to(dev), torch.randn(width, generator=g).to(dev)
    mix, w_out, w_in = torch.randn(streams, streams, generator=g).to(dev), torch.randn(streams, generator=g).to(dev), torch.randn(streams, generator=g).to(dev)
    old = h.clone()
    out = torch.empty(rows, width, dtype=dtype, device=dev)
    # write and read in one launch
    _call("streams", "mlr_streams_step", h.data_ptr(), y.data_ptr(), y.stride(0), scale.data_ptr(), mix.data_ptr(), w_out.data_ptr(),
          w_in.data_ptr(), norm_w.data_ptr(), 1e-5, out.data_ptr(), out.stride(0), native.is_bf16(out), None, rows, width, streams, native.stream())
    xs = old.double().cpu().view(rows, streams, width)
    new = plain.streams_write(xs, y.double().cpu() * scale.double().cpu(), mix.double().cpu(), w_out.double().cpu())
    assert torch.allclose(h.double().cpu().view(rows, streams, width), new, atol=1e-5, rtol=1e-5)
    want = plain.rms_norm(plain.streams_read(new, w_in.double().cpu()), norm_w.double().cpu(), 1e-5)
    tol = dict(atol=1e-4, rtol=1e-4) if dtype is torch.float32 else dict(atol=3e-2, rtol=2e-2)
    assert torch.allclose(out.double().cpu(), want, **tol)
    # the plain sum of chosen rows, normed (a model's last norm); the stream stays as it is
    chosen = torch.tensor([3, 0], dtype=torch.int32, device=dev)
    before = h.clone()
    out2 = torch.empty(2, width, dtype=dtype, device=dev)
    _call("streams", "mlr_streams_step", h.data_ptr(), None, 0, None, None, None, None, norm_w.data_ptr(), 1e-6, out2.data_ptr(), out2.stride(0),
          native.is_bf16(out2), chosen.data_ptr(), 2, width, streams, native.stream())
    want2 = plain.rms_norm(new[[3, 0]].sum(dim=1), norm_w.double().cpu(), 1e-6)
    assert torch.allclose(out2.double().cpu(), want2, **tol) and torch.equal(before, h)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,groups,keep,top,shared", [(8, 4, 2, 3, True), (6, 1, 1, 6, False), (5, 5, 2, 2, True), (12, 3, 1, 4, False),
                                                              (64, 8, 3, 8, True), (2, 2, 1, 1, False)])
def test_router_kernel(dtype, experts, groups, keep, top, shared):
    from mini_llm_runtime_b200.ops import native
    dev, rows, width = "cuda:0", 37, 24
    g = torch.Generator().manual_seed(experts)
    x = torch.randn(rows, width, generator=g).to(dtype).to(dev)
    router = torch.randn(experts + int(shared), width, generator=g).to(dev)
    correction = (torch.randn(experts, generator=g) - 1.0).to(dev)          # most choices below zero
    chosen = torch.empty(rows, top, dtype=torch.int32, device=dev)
    place = torch.empty_like(chosen)
    weights = torch.empty(rows, top, device=dev)
    gate = torch.empty(rows, device=dev)
    counts = torch.zeros(experts, dtype=torch.int32, device=dev)
    _call("experts", "mlr_experts_route", x.data_ptr(), x.stride(0), native.is_bf16(x), router.data_ptr(), correction.data_ptr(), rows, width,
          experts, groups, keep, top, int(shared), chosen.data_ptr(), weights.data_ptr(), place.data_ptr(), counts.data_ptr(),
          gate.data_ptr() if shared else None, 0, native.stream())
    xd = x.double().cpu()
    want_chosen, want_weights = plain.route(xd, router[:experts].double().cpu(), correction.double().cpu(), top, groups, keep)
    assert torch.equal(chosen.cpu().long(), want_chosen)
    assert torch.allclose(weights.double().cpu(), want_weights, atol=1e-5)
    if shared:
        assert torch.allclose(gate.double().cpu(), torch.sigmoid(xd @ router[experts].double().cpu()), atol=1e-5)
    assert counts.cpu().tolist() == torch.bincount(want_chosen.flatten(), minlength=experts).tolist()
    # a token's place among its expert's tokens: every expert's places are 0 .. count-1, each once
    for e in range(experts):
        mine = place.cpu()[chosen.cpu() == e]
        assert sorted(mine.tolist()) == list(range(len(mine)))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows", [1, 3, 70, 300])
def test_routed_experts_part_against_the_plain_function(dtype, rows):
    """The part by hand: route, arrange, both products over rows in the order by expert, combine, the shared expert."""
    from mini_llm_runtime_b200.config.base import PartSpec
    from mini_llm_runtime_b200.engine.runtime import Runtime
    from mini_llm_runtime_b200.parts.base import StepContext
    from mini_llm_runtime_b200.parts.experts import RoutedExperts
    from mini_llm_runtime_b200.csrc import build
    width, inter, experts, top, shared = 40, 24, 10, 3, 56
    g = torch.Generator().manual_seed(rows)
    names = {"router": "r", "correction": "c", "shared.gate": "sg.gate", "shared.up": "sg.up", "shared.down": "sg.down", "shared.sg": "sg.sg"}
    tensors = {"r": torch.randn(experts, width, generator=g), "c": torch.randn(experts, generator=g) * 0.3,
               "sg.gate": torch.randn(shared, width, generator=g) / 6, "sg.up": torch.randn(shared, width, generator=g) / 6,
               "sg.down": torch.randn(width, shared, generator=g) / 7, "sg.sg": torch.randn(1, width, generator=g)}
    for e in range(experts):
        for role, shape in (("gate", (inter, width)), ("up", (inter, width)), ("down", (width, inter))):
            names[f"e{e}.{role}"] = f"e{e}.{role}"
            tensors[f"e{e}.{role}"] = torch.randn(*shape, generator=g) / math.sqrt(shape[1])
    tensors = {k: v.bfloat16() for k, v in tensors.items()}
    rt = Runtime(torch.float32 if dtype == "float32" else torch.bfloat16)
    part = RoutedExperts(PartSpec("routed_experts", {"hidden_size": width, "intermediate_size": inter, "experts": experts, "top": top,
                                                     "groups": 5, "keep": 3, "shared_intermediate_size": shared}, names))
    build.ensure(part.kernel_modules(rt.dtype) + ["host"])
    part.bind(tensors, rt)
    x = torch.randn(rows, width, generator=g).to(rt.dtype).to(rt.device)
    status = torch.zeros(1, dtype=torch.int32, device=rt.device)
    step = StepContext(rt=rt, num_rows=rows, segments=[], token_ids=None, positions=None, segment_of_row=None, segment_info=None, slots=None,
                       tables={}, page_size=16, status=status)
    got = part.forward(x, step).double().cpu()
    got_again = part.forward(x, step).double().cpu()          # the counters are zero again after a step
    w = {"m." + k: v.double() for k, v in tensors.items()}
    w.update({"m.router": w["m.r"], "m.correction": w["m.c"]})
    w.update({"m.shared." + role: w["m.sg." + role] for role in ("gate", "up", "down", "sg")})
    mlp = {"router": {"experts": experts, "top": top, "groups": {"count": 5, "keep": 3}}, "shared": {"ff": shared}}
    want = plain.experts_feed_forward(x.double().cpu(), w, "m.", mlp)
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == "float32" else dict(atol=4e-2, rtol=4e-2)
    assert torch.allclose(got, want, **tol), float((got - want).abs().max())
    assert torch.equal(got, got_again)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,A,B,rows", [(3, 8, 24, 5), (1, 40, 130, 9), (20, 4, 12, 17), (2, 256, 64, 8)])
def test_per_head_projection_kernel(dtype, heads, A, B, rows):
    from mini_llm_runtime_b200.ops import native
    dev = "cuda:0"
    g = torch.Generator().manual_seed(A)
    x = torch.randn(rows, heads * A + 8, generator=g).to(dtype).to(dev)
    w = (torch.randn(heads, A, B, generator=g) / math.sqrt(A)).to(dtype).to(dev)
    y = torch.empty(rows, heads * B, dtype=dtype, device=dev)
    _call("latent", "mlr_head_project", x.data_ptr(), x.stride(0), w.data_ptr(), y.data_ptr(), y.stride(0), native.is_bf16(x), rows, heads, A, B,
          native.stream())
    want = torch.einsum("mha,hab->mhb", x[:, :heads * A].double().cpu().view(rows, heads, A), w.double().cpu()).reshape(rows, heads * B)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype is torch.float32 else dict(atol=2e-2, rtol=2e-2)
    assert torch.allclose(y.double().cpu(), want, **tol)


@pytest.mark.gpu
@pytest.mark.parametrize("heads,A,B,rows", [(3, 8, 24, 5), (2, 40, 130, 33), (16, 128, 64, 200), (1, 16, 8, 64), (4, 64, 256, 31)])
def test_per_head_projection_on_the_tensor_cores(heads, A, B, rows):
    """The bfloat16 form: one tensor-core product per head over all rows, matrices as [heads, outputs, inputs]."""
    from mini_llm_runtime_b200.ops import native
    dev = "cuda:0"
    g = torch.Generator().manual_seed(A + rows)
    x = torch.randn(rows, heads * A + 8, generator=g).bfloat16().to(dev)
    w = (torch.randn(heads, B, A, generator=g) / math.sqrt(A)).bfloat16().to(dev)
    y = torch.full((rows, heads * B + 3), float("nan"), dtype=torch.bfloat16, device=dev)
    _call("experts", "mlr_batched_product_bf16", x.data_ptr(), x.stride(0), w.data_ptr(), y.data_ptr(), y.stride(0), rows, heads, B, A, native.stream())
    want = torch.einsum("mha,hba->mhb", x[:, :heads * A].double().cpu().view(rows, heads, A), w.double().cpu()).reshape(rows, heads * B)
    assert torch.allclose(y[:, :heads * B].double().cpu(), want, atol=2e-2, rtol=2e-2)
    assert torch.isnan(y[:, heads * B:].float()).all()


def _latent_attention_case(dtype, heads, rank, T, page, loud=None, last_rows=None):
    """Latents of one request written into shuffled pages by `mlr_latent_cache`, then attention of every row (or of the
    last rows only) with the latents as keys and values of one shared kv head.  `loud`: a position whose latent is made
    to stand out for the last query."""
    from mini_llm_runtime_b200.ops import native
    from mini_llm_runtime_b200.ops.specs import GATES, MaskedAttentionSpec
    dev = "cuda:0"
    g = torch.Generator().manual_seed(T + rank)
    q = torch.randn(T, heads * rank, generator=g)
    down = torch.randn(T, rank + 5, generator=g)
    weight = (1.0 + 0.2 * torch.randn(rank, generator=g)).to(dev)
    if loud is not None:
        down[loud, :rank] = 0.0
        down[loud, 1] = 50.0                      # after the norm: one large value
        q[T - 1] = 0.0
        q[T - 1].view(heads, rank)[:, 1] = 30.0
    q, down = q.to(dtype).to(dev), down.to(dtype).to(dev)
    n_pages = (T + page - 1) // page + 2
    order = torch.randperm(n_pages, generator=g)[:(T + page - 1) // page].to(torch.int32)
    table = order.reshape(1, -1).to(dev)
    cache = torch.full((n_pages, page * rank), float("nan"), dtype=dtype, device=dev)
    positions, of_row, info = _meta([(0, T, 0, 0)], dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    _call("latent", "mlr_latent_cache", down.data_ptr(), down.stride(0), native.is_bf16(down), weight.data_ptr(), 1, 1e-5, rank, cache.data_ptr(),
          n_pages, positions.data_ptr(), of_row.data_ptr(), table.data_ptr(), table.stride(0), page, T, status.data_ptr(), native.stream())
    c = plain.rms_norm(down[:, :rank].double().cpu(), weight.double().cpu(), 1e-5)
    stored = torch.stack([cache[int(order[t // page])].view(page, rank)[t % page] for t in range(T)]).double().cpu()
    assert torch.allclose(stored, c, atol=1e-5 if dtype is torch.float32 else 3e-2, rtol=1e-5 if dtype is torch.float32 else 1e-2)
    spec = MaskedAttentionSpec(freq=None, heads=heads, kv_heads=1, dim=rank, vdim=rank, rot_dims=0, window=0, chunk=0, sink=0,
                               gate_kind=GATES[None], shared_kv=1, scale=0.15, out_scale=1.0)
    out = torch.full((T, heads * rank), float("nan"), dtype=dtype, device=dev)
    _call("attention_masked", "mlr_attention_masked", ctypes.addressof(spec), q.data_ptr(), q.stride(0), None, 0, out.data_ptr(), out.stride(0),
          native.is_bf16(q), cache.data_ptr(), n_pages, positions.data_ptr(), of_row.data_ptr(), table.data_ptr(), table.stride(0), page, T, None,
          0, None, 0, 1, 1, None, status.data_ptr(), native.stream())
    if last_rows:       # as a step of decoded tokens runs: the last rows as a segment of few rows, its keys cut into ranges that a
        rows, keys, most = last_rows                                       # second kernel adds up
        segment = torch.tensor([[T - rows, rows, T - rows, 0]], dtype=torch.int32, device=dev)
        partial = torch.full((16 * most * (rank + 2),), float("nan"), device=dev)
        cut = torch.full((T, heads * rank), float("nan"), dtype=dtype, device=dev)
        _call("attention_masked", "mlr_attention_masked", ctypes.addressof(spec), q.data_ptr(), q.stride(0), None, 0, cut.data_ptr(), cut.stride(0),
              native.is_bf16(q), cache.data_ptr(), n_pages, positions.data_ptr(), of_row.data_ptr(), table.data_ptr(), table.stride(0), page, 0, None,
              1, segment.data_ptr(), keys, most, 1, partial.data_ptr(), status.data_ptr(), native.stream())
        out[T - rows:] = cut[T - rows:]
    tiled = None
    if dtype is torch.bfloat16 and rank % 16 == 0 and rank <= 128:
        tiled = torch.full((T, heads * rank), float("nan"), dtype=dtype, device=dev)
        tiles = torch.tensor([(0, t) for t in range(0, T, 64)], dtype=torch.int32, device=dev)
        _call("attention_masked", "mlr_attention_masked_tiles", ctypes.addressof(spec), q.data_ptr(), q.stride(0), None, 0, tiled.data_ptr(),
              tiled.stride(0), cache.data_ptr(), n_pages, tiles.data_ptr(), tiles.shape[0], info.data_ptr(), table.data_ptr(), table.stride(0),
              page, status.data_ptr(), native.stream())
    assert int(status.item()) == 0
    qd = q.double().cpu().view(T, heads, rank)
    seen = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    want = torch.zeros(T, heads, rank, dtype=torch.float64)
    for h in range(heads):
        s = (qd[:, h] @ stored.T) * 0.15
        want[:, h] = torch.softmax(s.masked_fill(~seen, -math.inf), dim=-1) @ stored
    return out.double().cpu(), tiled.double().cpu() if tiled is not None else None, want.reshape(T, heads * rank), stored


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,rank,T,page", [(4, 16, 150, 8), (20, 12, 40, 16), (2, 64, 300, 16), (1, 256, 70, 4), (2, 520, 45, 8), (1, 1024, 20, 16)])
def test_attention_on_cached_latents(dtype, heads, rank, T, page):
    got, tiled, want, _ = _latent_attention_case(dtype, heads, rank, T, page)
    tol = dict(atol=1e-4, rtol=1e-4) if dtype is torch.float32 else dict(atol=3e-2, rtol=3e-2)
    assert torch.allclose(got, want, **tol)
    if tiled is not None:
        assert torch.allclose(tiled, want, **tol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,page,loud", [(700, 16, 0), (700, 16, 1), (513, 16, 15), (513, 16, 16), (513, 8, 247), (400, 16, 399), (400, 16, 398)])
def test_one_loud_latent_far_back_or_at_a_page_border_takes_the_weight(dtype, T, page, loud):
    """Among hundreds of latents one is made to stand out for the last query: its row is what comes out, wherever it
    lies (the first tokens, a page's last or first place, the query itself)."""
    got, tiled, want, stored = _latent_attention_case(dtype, 3, 32, T, page, loud=loud)
    for have in (got, tiled):
        if have is None:
            continue
        last = have[T - 1].view(3, 32)
        assert torch.allclose(last, stored[loud].expand(3, 32), atol=2e-2, rtol=2e-2)
        assert torch.allclose(have, want, atol=3e-2, rtol=3e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,page,loud,rows", [(700, 16, 0, 1), (700, 16, 1, 1), (641, 16, 63, 1), (641, 16, 64, 2), (700, 8, 639, 1), (700, 16, 699, 1),
                                               (700, 16, 698, 2)])
def test_one_loud_latent_for_a_decoded_token_whose_keys_are_cut_into_ranges(dtype, T, page, loud, rows):
    """The same for the last rows run as a decode step runs them: key ranges of 64 as blocks of their own, added up by the merge
    kernel; the loud latent at the first places, at a range's last and first place, in the last range."""
    got, _, want, stored = _latent_attention_case(dtype, 3, 32, T, page, loud=loud, last_rows=(rows, 64, 12))
    assert torch.allclose(got[T - 1].view(3, 32), stored[loud].expand(3, 32), atol=2e-2, rtol=2e-2)
    assert torch.allclose(got, want, atol=3e-2, rtol=3e-2)


# ----------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module", params=sorted(niridra_models.ALL))
def case(request, tmp_path_factory):
    config = niridra_models.get(request.param)
    weights = niridra_models.random_weights(config, seed=11)
    folder = str(tmp_path_factory.mktemp(request.param))
    write_model_folder(folder, config, weights)
    return folder, config, weights


def close(got, want, dtype, what):
    """float32: every value.  bfloat16: row by row, and a few rows may be off altogether: where two experts' choice scores
    are nearly equal, the rounding of the router's input lets the choice fall the other way, and that row (and what later
    rows read of it) then differs by an expert's whole output.  The float32 runs of the same tests allow no such row."""
    if dtype != "bfloat16":
        return assert_close(got, want, dtype, what)
    from helpers import row_metrics
    assert got.shape == want.shape and torch.isfinite(got).all(), what
    m = row_metrics(got, want)
    bad = (m["rmse"] > BF16["rmse"]) | (m["max"] > BF16["max"]) | (m["cosine"] < BF16["cosine"])
    allowed = max(2, got.shape[0] // 25)
    assert int(bad.sum()) <= allowed, (f"{what}: {int(bad.sum())} of {bad.numel()} rows are off (a router's close calls explain up to {allowed}); "
                                       f"worst: rmse {m['rmse'].max():.4f}, max {m['max'].max():.4f}, cosine {m['cosine'].min():.6f}")


@pytest.mark.gpu
def test_every_layer_of_a_short_prompt(case):
    """The sum of the stream's copies after every layer, float32, with the steps driven from Python part by part."""
    from mini_llm_runtime_b200.engine.model import StepEntry
    folder, config, weights = case
    model = engine_model(folder, "float32", num_pages=8, page_size=8, max_requests=1)
    model._native = None
    S, W = config.get("streams") or 1, config["width"]
    seen = []
    for run in model.runs:
        def wrapped(h, pending, step, ctx, inner=run.block.forward):
            result = inner(h, pending, step, ctx)
            seen.append(h.view(h.shape[0], S, W).sum(dim=1).double().cpu())
            return result
        run.block.forward = wrapped
    tokens = tokens_for(config, 19, 2)
    slot = model.open_request()
    model.step([StepEntry(slot, tokens, [18])])
    want = []
    plain.forward(config, {k: v.double() for k, v in weights.items()}, tokens, want)
    assert len(seen) == len(want)
    for i, (a, b) in enumerate(zip(seen, want)):
        assert torch.allclose(a, b, atol=2e-4, rtol=2e-4), i


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
    # Three live requests at a time; a finished one gives its slot (with the state of its mixers and the token the
    # embedding kept) and its pages to the next.
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
def test_long_decoding_through_the_graphs_keeps_the_state_right(case):
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
