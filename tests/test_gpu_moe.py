"""GPU parity of the MoE expert path (router, routing, grouped W6A8 GEMMs with the SwiGLU
epilogue, combine) through the C ABI, against the oracle. Bar: rtol = atol = 0.03
(tests/native_mxfp6/test_moe.py:248) and relative Frobenius error <= 1e-2; routing tables
checked exactly."""
import pytest
import torch

from oracle import mx_oracle as ora
from tests.gpu_util import gpu_available, randn_bf16, rel_fro

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not gpu_available(), reason="needs a B200")]


@pytest.fixture(scope="module")
def nat():
    from mach_b200 import native
    native.lib()
    return native


def make_experts(experts, hidden, inter, seed, fmt):
    g = torch.Generator().manual_seed(seed)
    w13 = (0.05 * torch.randn(experts, 2 * inter, hidden, generator=g)).to(torch.bfloat16)
    w2 = (0.05 * torch.randn(experts, hidden, inter, generator=g)).to(torch.bfloat16)
    if fmt == "e4m3":
        q13 = [ora.quantize_weight_mxfp8(w13[e]) for e in range(experts)]
        q2 = [ora.quantize_weight_mxfp8(w2[e]) for e in range(experts)]
        pack = lambda c: c
        deq = ora.dequantize_mx
    else:
        q13 = [ora.quantize_weight_mxfp6(w13[e], fmt) for e in range(experts)]
        q2 = [ora.quantize_weight_mxfp6(w2[e], fmt) for e in range(experts)]
        pack = ora.pack_fp6
        deq = lambda c, s: ora.dequantize_mxfp6(c, s, fmt)
    c13 = torch.stack([pack(c) for c, _ in q13]); s13 = torch.stack([s for _, s in q13])
    c2 = torch.stack([pack(c) for c, _ in q2]); s2 = torch.stack([s for _, s in q2])
    w13_deq = lambda e: deq(*q13[e])
    w2_deq = lambda e: deq(*q2[e])
    return (c13, s13, c2, s2), w13_deq, w2_deq


@pytest.mark.parametrize("m,experts,top_k", [(1, 256, 8), (64, 256, 8), (7, 8, 2), (300, 32, 4)])
def test_router_topk(nat, m, experts, top_k):
    from mach_b200 import moe
    logits = randn_bf16(m, experts, 7000 + m)
    w, ids = moe.router_topk(logits.cuda(), top_k)
    ref_w, ref_ids = ora.route_topk(logits, top_k)
    probs = torch.softmax(logits.float(), -1)
    picked = probs.gather(1, ids.cpu().long())
    # BF16 logits tie often: the selected probabilities must match, ids may differ at ties.
    assert torch.allclose(picked.sort(-1).values, probs.gather(1, ref_ids.long()).sort(-1).values)
    assert torch.allclose(w.cpu(), picked / picked.sum(-1, keepdim=True), rtol=1e-5, atol=1e-7)
    assert bool((ids.cpu().sort(-1).values.diff(dim=-1) != 0).all())  # distinct experts


@pytest.mark.parametrize("m,experts,hidden,inter,top_k,fmt,ep", [
    (1, 16, 256, 128, 4, "e4m3", None), (16, 16, 256, 128, 4, "e2m3", None),
    (33, 8, 512, 256, 2, "e3m2", None), (200, 8, 256, 128, 2, "e2m3", None),
    (64, 32, 256, 128, 8, "e2m3", (1, 2)), (700, 4, 256, 128, 2, "e4m3", None),
    (300, 4, 384, 192, 2, "e4m3", None), (512, 8, 512, 256, 2, "e2m3", None),
    (1000, 16, 256, 128, 4, "e3m2", (0, 2)),
])
def test_experts_forward(nat, m, experts, hidden, inter, top_k, fmt, ep):
    from mach_b200 import moe
    x = randn_bf16(m, hidden, 8000 + m)
    logits = randn_bf16(m, experts, 8001 + m)
    (c13, s13, c2, s2), w13_deq, w2_deq = make_experts(experts, hidden, inter, 8002 + m, fmt)
    topk_w, topk_ids = moe.router_topk(logits.cuda(), top_k)
    expert_map = None
    local = range(experts)
    if ep is not None:  # expert parallel: this rank holds a contiguous slice of the experts
        rank, world = ep
        per = experts // world
        local = range(rank * per, (rank + 1) * per)
        expert_map = torch.full((experts,), -1, dtype=torch.int32)
        expert_map[rank * per:(rank + 1) * per] = torch.arange(per, dtype=torch.int32)
    sel = list(local)
    weights = moe.MoeWeights.from_logical(c13[sel].cuda(), s13[sel].cuda(), c2[sel].cuda(),
                                          s2[sel].cuda(), fmt)
    out = moe.experts_forward(x.cuda(), weights, topk_w, topk_ids,
                              None if expert_map is None else expert_map.cuda())
    torch.cuda.synchronize()
    assert nat.device_status() == 0
    ref = ora.moe_forward(x, lambda e: w13_deq(sel[e]), lambda e: w2_deq(sel[e]), topk_w.cpu(),
                          topk_ids.cpu(), expert_map)
    assert torch.isfinite(out.float()).all()
    assert torch.allclose(out.float().cpu(), ref.float(), rtol=0.03, atol=0.03)
    assert rel_fro(out, ref) <= 1e-2


def test_moe_config5_shape_decode(nat):
    """Benchmark configuration 5 geometry (256 experts, top-8, hidden 2048, intermediate 512, E2M3)
    at M = 64; only the experts actually hit are dequantised by the oracle."""
    from mach_b200 import moe
    m, experts, hidden, inter, top_k = 64, 256, 2048, 512, 8
    x = randn_bf16(m, hidden, 1)
    logits = randn_bf16(m, experts, 2)
    g = torch.Generator().manual_seed(3)
    codes13 = torch.randint(0, 64, (experts, 2 * inter, hidden), generator=g, dtype=torch.uint8)
    codes2 = torch.randint(0, 64, (experts, hidden, inter), generator=g, dtype=torch.uint8)
    s13 = torch.randint(116, 120, (experts, 2 * inter, hidden // 32), generator=g, dtype=torch.uint8)
    s2 = torch.randint(116, 120, (experts, hidden, inter // 32), generator=g, dtype=torch.uint8)
    pack = lambda c: torch.stack([ora.pack_fp6(c[e]) for e in range(c.shape[0])])
    weights = moe.MoeWeights.from_logical(pack(codes13).cuda(), s13.cuda(), pack(codes2).cuda(),
                                          s2.cuda(), "e2m3")
    topk_w, topk_ids = moe.router_topk(logits.cuda(), top_k)
    out = moe.experts_forward(x.cuda(), weights, topk_w, topk_ids)
    torch.cuda.synchronize()
    assert nat.device_status() == 0
    ref = ora.moe_forward(x, lambda e: ora.dequantize_mxfp6(codes13[e], s13[e], "e2m3"),
                          lambda e: ora.dequantize_mxfp6(codes2[e], s2[e], "e2m3"),
                          topk_w.cpu(), topk_ids.cpu())
    assert torch.allclose(out.float().cpu(), ref.float(), rtol=0.03, atol=0.03)
    assert rel_fro(out, ref) <= 1e-2


@pytest.mark.parametrize("m,experts,top_k,hidden", [(1, 16, 4, 256), (77, 8, 2, 512), (300, 32, 8, 2048)])
def test_scatter_quantize_equals_gather_quantize(nat, m, experts, top_k, hidden):
    """The token-major quantise + scatter writes, for every live permuted row, the bytes the
    row-major gather + quantise writes (same arithmetic per token)."""
    from mach_b200 import moe
    lib = nat.lib()
    x = randn_bf16(m, hidden, 8800 + m).cuda()
    logits = randn_bf16(m, experts, 8801 + m).cuda()
    _, ids = moe.router_topk(logits, top_k)
    chunk = moe.chunk_rows_for(m, top_k, experts)
    rows_cap = int(lib.mach_moe_rows_cap(m, top_k, experts))
    work_cap = int(lib.mach_moe_work_cap(m, top_k, experts, chunk))
    i32 = dict(dtype=torch.int32, device="cuda")
    counts, offsets = torch.empty(experts, **i32), torch.empty(experts + 1, **i32)
    pos_of, src_of = torch.empty(m * top_k, **i32), torch.full((rows_cap,), -1, **i32)
    work, num_work = torch.empty(3 * work_cap, **i32), torch.empty(1, **i32)
    p, st = nat._ptr, nat._stream(x)
    nat._check(lib.mach_moe_route(p(ids), None, m, top_k, experts, chunk, rows_cap, work_cap,
                                  p(counts), p(offsets), p(pos_of), p(src_of), p(work), p(num_work),
                                  st), "route")
    outs = []
    for which in ("gather", "scatter"):
        codes = torch.zeros((rows_cap, hidden), dtype=torch.uint8, device="cuda")
        scales = torch.zeros(nat.sf_bytes(rows_cap, hidden), dtype=torch.uint8, device="cuda")
        if which == "gather":
            nat._check(lib.mach_moe_gather_quantize(p(x), p(src_of), p(offsets), experts, rows_cap,
                                                    hidden, p(codes), p(scales), st), which)
        else:
            nat._check(lib.mach_moe_scatter_quantize(p(x), p(pos_of), m, top_k, hidden, p(codes),
                                                     p(scales), st), which)
        outs.append((codes, nat.unpack_scales(scales, rows_cap, hidden)))
    torch.cuda.synchronize()
    total = int(offsets[-1])
    live = (src_of[:total] >= 0).nonzero().flatten()
    assert live.numel() == m * top_k
    assert torch.equal(outs[0][0][live], outs[1][0][live])
    assert torch.equal(outs[0][1][live], outs[1][1][live])


@pytest.mark.parametrize("m,experts,hidden,inter,top_k,fmt,ep", [
    (1, 16, 256, 128, 4, "e4m3", None), (1, 256, 2048, 512, 8, "e2m3", None),
    (2, 8, 512, 256, 2, "e3m2", None), (4, 32, 2048, 512, 8, "e2m3", (1, 2)),
    (8, 16, 384, 256, 4, "e2m3", None), (8, 64, 256, 128, 8, "e4m3", (3, 4)),
])
def test_small_batch_schedule(nat, m, experts, hidden, inter, top_k, fmt, ep):
    """The decode schedule (mach_moe_small_batch, M <= 8) against the oracle and against the
    grouped tensor-core path on the same inputs. Same rounding points, another summation
    order inside the dot products: the layer's tolerance applies (rtol = atol = 0.03)."""
    from mach_b200 import moe
    x = randn_bf16(m, hidden, 8400 + m)
    logits = randn_bf16(m, experts, 8401 + m)
    (c13, s13, c2, s2), w13_deq, w2_deq = make_experts(min(experts, 16), hidden, inter, 8402 + m, fmt)
    base = c13.shape[0]
    pick = [e % base for e in range(experts)]          # bounded CPU work: experts repeat modulo 16
    shift = torch.tensor([(e // base) % 3 for e in range(experts)], dtype=torch.uint8)
    c13, c2 = c13[pick], c2[pick]
    s13 = s13[pick] + shift[:, None, None]
    s2 = s2[pick] + shift[:, None, None]
    d13 = lambda e: w13_deq(e % base) * 2.0 ** int(shift[e])
    d2 = lambda e: w2_deq(e % base) * 2.0 ** int(shift[e])
    topk_w, topk_ids = moe.router_topk(logits.cuda(), top_k)
    expert_map, sel = None, list(range(experts))
    if ep is not None:
        rank, world = ep
        per = experts // world
        sel = list(range(rank * per, (rank + 1) * per))
        expert_map = torch.full((experts,), -1, dtype=torch.int32)
        expert_map[rank * per:(rank + 1) * per] = torch.arange(per, dtype=torch.int32)
    weights = moe.MoeWeights.from_logical(c13[sel].cuda(), s13[sel].cuda(), c2[sel].cuda(),
                                          s2[sel].cuda(), fmt)
    emap = None if expert_map is None else expert_map.cuda()
    limit = moe.SMALL_BATCH_MAX_TOKENS
    try:
        moe.SMALL_BATCH_MAX_TOKENS = 8          # the entry point's own limit
        small = moe.experts_forward(x.cuda(), weights, topk_w, topk_ids, emap)
        moe.SMALL_BATCH_MAX_TOKENS = 0
        grouped = moe.experts_forward(x.cuda(), weights, topk_w, topk_ids, emap)
    finally:
        moe.SMALL_BATCH_MAX_TOKENS = limit
    torch.cuda.synchronize()
    assert nat.device_status() == 0
    ref = ora.moe_forward(x, lambda e: d13(sel[e]), lambda e: d2(sel[e]), topk_w.cpu(),
                          topk_ids.cpu(), expert_map)
    assert torch.isfinite(small.float()).all()
    assert torch.allclose(small.float().cpu(), ref.float(), rtol=0.03, atol=0.03), \
        float((small.float().cpu() - ref.float()).abs().max())
    assert torch.allclose(small.float(), grouped.float(), rtol=0.03, atol=0.03)
    assert rel_fro(small, ref) <= 1e-2


def test_small_batch_refuses_what_it_does_not_implement(nat):
    import ctypes
    lib = nat.lib()
    d = torch.zeros(64, dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [d.data_ptr()] * 10
    assert lib.mach_moe_small_batch(*args, 9, 8, 256, 2048, 512, 3, stream) == 2      # M > 8
    assert lib.mach_moe_small_batch(*args, 1, 8, 256, 2000, 512, 3, stream) == 2      # hidden % 128
    assert lib.mach_moe_small_batch(*args, 1, 8, 256, 2048, 512, 7, stream) == 1      # format
    assert lib.mach_moe_small_batch(*args, 0, 8, 256, 2048, 512, 3, stream) == 0      # empty batch
    assert lib.mach_moe_small_scratch_bytes(1, 8, 2048, 512) == 2048 * 4 + 8 * 512 * 4 + 8 * 4
