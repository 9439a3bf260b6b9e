"""The kernels the Vokepel design added, each alone against a plain PyTorch reference in float64 (GPU)."""
import math

import pytest
import torch

from test_gpu_kernels import DEV, paged_case, rel, rnd

pytestmark = pytest.mark.gpu


def talking_reference(case, HQ, HKV, D, window, scale, cap, slope, rate, talk, sink, gate):
    """Per request and row: all heads' scores, capped, biased by the distance, mixed, then a softmax with a sink."""
    out = torch.zeros(case["T"], HQ, D, dtype=torch.float64)
    f = lambda t: None if t is None else t.double().cpu()
    slope, rate, talk, sink, gate = f(slope), f(rate), f(talk), f(sink), f(gate)
    row = 0
    for (ctx, ql), (k, v) in zip(case["segs"], case["dense"]):
        k, v = k.double().cpu(), v.double().cpu()
        for i in range(ql):
            z = ctx - ql + i
            lo = max(0, z - window + 1) if window else 0
            q = case["q"][row].double().cpu()                                     # [HQ, D]
            kk = k[lo:z + 1].repeat_interleave(HQ // HKV, dim=1)                     # [n, HQ, D]
            s = torch.einsum("hd,nhd->hn", q, kk) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            if slope is not None:
                dist = (z - torch.arange(lo, z + 1)).double()
                s = s - slope[:, None] * torch.log1p(rate[:, None] * dist[None])
            if talk is not None:
                s = talk @ s
            top = s.max(dim=1, keepdim=True).values
            if sink is not None:
                top = torch.maximum(top, sink[:, None])
            e = torch.exp(s - top)
            den = e.sum(dim=1, keepdim=True) + (torch.exp(sink[:, None] - top) if sink is not None else 0.0)
            o = torch.einsum("hn,nhd->hd", e / den, v[lo:z + 1].repeat_interleave(HQ // HKV, dim=1))
            if gate is not None:
                o = o * torch.sigmoid(gate[row].view(HQ, D))
            out[row] = o
            row += 1
    return out.view(case["T"], HQ * D)


def extras(HQ, D, T, dtype, seed, with_all=True):
    g = torch.Generator().manual_seed(seed)
    slope = (torch.randn(HQ, generator=g) * 0.4).to(DEV)
    rate = (torch.rand(HQ, generator=g) * 1.5 + 0.05).to(DEV)
    talk = (torch.eye(HQ) + 0.3 * torch.randn(HQ, HQ, generator=g)).to(DEV)
    sink = (torch.randn(HQ, generator=g) * 1.5).to(DEV)
    gate = torch.randn(T, HQ * D, generator=g).to(dtype).to(DEV)
    return slope, rate, talk, sink, gate


@pytest.mark.parametrize("HQ,HKV,D,page_size,window,cap", [
    (4, 2, 16, 16, None, 5.0), (6, 3, 48, 8, 24, 20.0), (3, 1, 80, 5, 7, 0.0), (12, 4, 32, 16, 100, 3.0), (1, 1, 40, 16, 33, 8.0),
    (36, 6, 8, 16, 50, 4.0), (64, 16, 16, 8, None, 9.0)])            # two and four heads per warp
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_talking_plain_kernel(HQ, HKV, D, page_size, window, cap, dtype):
    from purhie_b200.csrc import ops
    segs = [(1, 1), (33, 33), (70, 1), (129, 17), (40, 2)]
    case = paged_case(segs, HQ, HKV, D, page_size, dtype, seed=3)
    scale = 2.0 / math.sqrt(D)
    slope, rate, talk, sink, gate = extras(HQ, D, case["T"], dtype, 7)
    kw = dict(num_heads=HQ, num_kv_heads=HKV, head_dim=D, window=window, scale=scale)
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    for use in ({"cap": cap, "slope": slope, "rate": rate, "talk": talk, "sink": sink, "gate": gate}, {"cap": cap, "talk": talk},
                {"slope": slope, "rate": rate}, {"sink": sink}, {}):
        out = torch.full((case["T"], HQ * D), float("nan"), dtype=dtype, device=DEV)
        ops.attention_talking(case["q"], case["k_base"], case["v_base"], case["page_stride"], page_size, case["table"], case["row_seg"],
                              case["positions"], out, **kw, **use)
        ref = talking_reference(case, HQ, HKV, D, window, scale, use.get("cap", 0.0), use.get("slope"), use.get("rate"), use.get("talk"),
                                use.get("sink"), use.get("gate"))
        assert rel(out.cpu(), ref) < tol
    # the plain attention kernel with a sink agrees with the same reference
    out = torch.full((case["T"], HQ * D), float("nan"), dtype=dtype, device=DEV)
    ops.attention_generic_sink(case["q"], case["k_base"], case["v_base"], case["page_stride"], page_size, case["table"], case["row_seg"],
                               case["positions"], out, sink, **kw)
    assert rel(out.cpu(), talking_reference(case, HQ, HKV, D, window, scale, 0.0, None, None, None, sink, None)) < tol


@pytest.mark.parametrize("HQ,HKV,D,page_size,window,cap", [
    (4, 2, 16, 16, None, 5.0), (6, 3, 48, 8, 24, 20.0), (16, 4, 128, 16, 150, 30.0), (8, 1, 64, 32, 77, 0.0), (5, 5, 96, 8, 40, 6.0),
    (32, 8, 32, 16, 90, 10.0), (24, 2, 64, 16, None, 4.0)])
def test_attention_talking_tile_kernel(HQ, HKV, D, page_size, window, cap):
    """Tiles of 16 rows: portions that start mid-page and end inside a tile, decode rows short and long, keys shared by
    one, three and more CTAs than a tile has blocks; two equally good keys either side of the window's edge are told apart
    by the reference itself."""
    from purhie_b200.csrc import ops
    assert ops.attention_talking_mma_supports(HQ, HKV, D, D)
    segs = [(1, 1), (64, 64), (200, 130), (300, 1), (65, 2), (513, 97), (63, 1), (128, 1)]
    case = paged_case(segs, HQ, HKV, D, page_size, torch.bfloat16, seed=4)
    scale = 2.0 / math.sqrt(D)
    slope, rate, talk, sink, gate = extras(HQ, D, case["T"], torch.bfloat16, 9)
    tiles = [(s, f) for s, (ctx, ql) in enumerate(segs) for f in range(0, ql, 16)]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    tile_seg, tile_first = i32([t[0] for t in tiles]), i32([t[1] for t in tiles])
    kw = dict(num_heads=HQ, num_kv_heads=HKV, head_dim=D, window=window, scale=scale)
    for use in ({"cap": cap, "slope": slope, "rate": rate, "talk": talk, "sink": sink, "gate": gate}, {"sink": sink}, {"cap": cap, "talk": talk}):
        ref = talking_reference(case, HQ, HKV, D, window, scale, use.get("cap", 0.0), use.get("slope"), use.get("rate"), use.get("talk"),
                                use.get("sink"), use.get("gate"))
        for splits in (1, 3, 24):
            out = torch.full((case["T"], HQ * D), float("nan"), dtype=torch.bfloat16, device=DEV)
            ops.attention_talking_mma(case["q"], case["k_base"], case["v_base"], case["page_stride"], page_size, case["table"],
                                      case["seg_start"], case["seg_ctx"], tile_seg, tile_first, out, splits=splits, **kw, **use)
            assert not torch.isnan(out.float()).any()
            assert rel(out.cpu(), ref) < 1.2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_min_gru_scan_rows_and_chunks(dtype):
    from purhie_b200.csrc import ops
    W, lens, slots = 72, [1, 150, 7, 33], [2, 0, 3, 1]
    T = sum(lens)
    rows = rnd(2, T, 3 * W, dtype=dtype, seed=1)                                       # two partial sums
    zb, xb = rnd(W, seed=2, scale=0.5), rnd(W, seed=3, scale=0.5)
    state0 = rnd(4, W, seed=4)
    a = rows.double().sum(0).cpu()
    ref, ref_state, at = torch.zeros(T, W, dtype=torch.float64), state0.double().cpu().clone(), 0
    for n, slot in zip(lens, slots):
        s = ref_state[slot].clone()
        for t in range(at, at + n):
            z, u, g = torch.sigmoid(a[t, :W] + zb.double().cpu()), a[t, W:2 * W] + xb.double().cpu(), a[t, 2 * W:]
            cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
            s = (1 - z) * s + z * cand
            ref[t] = s * g * torch.sigmoid(g)
        ref_state[slot] = s
        at += n
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    seg_start = i32([0] + list(torch.tensor(lens).cumsum(0)))
    chunks, seg_chunks, row = [], [0], 0
    for s, n in enumerate(lens):
        for c in range(0, n, 32):
            chunks += [row + c, min(32, n - c), s, int(c + 32 >= n)]
        row += n
        seg_chunks.append(len(chunks) // 4)
    for use_chunks in (False, True):
        state = state0.clone()
        out = torch.full((T, W), float("nan"), dtype=dtype, device=DEV)
        ops.min_gru_scan(rows, zb, xb, state, seg_start, i32(slots), out, i32(chunks) if use_chunks else None, i32(seg_chunks) if use_chunks else None)
        assert rel(out.cpu(), ref) < (3e-6 if dtype == torch.float32 else 8e-3)
        assert rel(state.cpu(), ref_state) < 3e-6


def test_pair_sum_scale_softcap_and_the_norm_with_a_factor_on_its_addend():
    from purhie_b200.csrc import ops
    T, E = 37, 200
    a, b = rnd(3, T * E, dtype=torch.bfloat16, seed=1), rnd(1, T * E, seed=2)
    out = torch.empty(T * E, dtype=torch.float32, device=DEV)
    ops.pair_sum(a, 0.8, b, -1.3, out)
    assert rel(out.cpu(), 0.8 * a.double().sum(0).cpu() - 1.3 * b.double().sum(0).cpu()) < 1e-6
    y = rnd(5, 333, seed=3, scale=20.0)
    ref = 12.0 * torch.tanh(y.double().cpu() * 1.7 / 12.0)
    assert rel(ops.scale_softcap(y.clone(), 1.7, 12.0).cpu(), ref) < 1e-6
    assert rel(ops.scale_softcap(y.clone(), 0.5, 0.0).cpu(), 0.5 * y.double().cpu()) < 1e-6
    for E2, splits in ((200, 3), (4096, 9), (5120, 1), (50, 2)):
        x, add, w = rnd(T, E2, seed=4), rnd(splits, T, E2, dtype=torch.bfloat16, seed=5), rnd(E2, seed=6) + 1.0
        v = x.double().cpu() + 0.6 * add.double().sum(0).cpu()
        ref_y = v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-5) * w.double().cpu()
        yy = torch.empty(T, E2, dtype=torch.bfloat16, device=DEV)
        ops.add_scaled_rmsnorm(x, add, w, 1e-5, yy, 0.6, add_splits=splits)
        assert rel(x.cpu(), v) < 1e-6 and rel(yy.cpu(), ref_y) < 8e-3
