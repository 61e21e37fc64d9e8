"""Worker of the multi-GPU tests; started by tests/test_fused_multi_gpu.py through
``python -m torch.distributed.run``. Every rank uses different, seeded data. Prints one JSON
line per case on rank 0 and exits non-zero if any rank saw a failure."""
import json
import os
import sys

import torch
import torch.distributed as dist

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)

import mm_rs_with_catlass_b200 as catcoc  # noqa: E402
from mm_rs_with_catlass_b200.ops import reference as ref  # noqa: E402
from mm_rs_with_catlass_b200.utils.data import matmul_inputs, quant_inputs  # noqa: E402
from mm_rs_with_catlass_b200.utils.verify import verify  # noqa: E402

rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)
mode = sys.argv[1] if len(sys.argv) > 1 else "ops"
failures = []


def pmag(*args, **kw):
    """Error scale of a sum of partial results that were rounded before they were added
    (``reference.partial_magnitude``). Where the heap has a multicast alias the default data path
    adds the partials inside NVSwitch, whose bf16 / fp16 result can be a whole unit in the last
    place away from the exact sum of the rounded partials (a round-to-nearest adder, as in the
    owner-side sum of the push flavour, stays within half a unit): the bound grows from
    u (sum |partial| + |sum|) to u (sum |partial| + 2 |sum|) <= 1.5 x the former."""
    m = ref.partial_magnitude(*args, **kw)
    c = catcoc.parallel.shmem._default_ctx
    return m * 1.5 if (c is not None and c.multicast) else m


def agree(ok: bool) -> bool:
    t = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item())


def report(name, ok, detail=""):
    ok_all = agree(ok)
    if not ok_all:
        failures.append(name)
    if rank == 0:
        print(json.dumps({"case": name, "ok": ok_all, "detail": detail if not ok else ""}), flush=True)


def check(name, out, gold, k, dtype, magnitude=None):
    r = verify(out, gold, k, dtype, magnitude)
    try:
        ctx.check(name)
        st = ""
    except RuntimeError as e:
        st = str(e)
    report(name, r.ok and not st, "%s %s" % (r, st))


def run_mixed_launches(ctx, W, iters, name):
    """Many back-to-back launches of mixed ops on one context (epoch parity, stamp and slab reuse):
    every result is checked, so a launch that raced with its neighbours shows up as a wrong tile."""
    a, b = matmul_inputs(128 * W, 256, 128, rank, torch.bfloat16, dev, seed=77)
    gold = ref.matmul_allreduce(a, b, out_dtype=torch.float32)
    mag = pmag(a, b)
    rows = 128
    ok = True
    bad = []
    ag_gold = None
    for it in range(iters):
        if it % 3 == 0:
            o = catcoc.matmul_reduce_scatter(a, b)
            r = verify(o, gold[rank * rows:(rank + 1) * rows], 128 * W, torch.bfloat16, mag[rank * rows:(rank + 1) * rows])
            if not r.ok:
                bad.append("it %d rs rank %d: %s" % (it, rank, r))
        elif it % 3 == 1:
            o = catcoc.matmul_allreduce(a, b).clone()
            r = verify(o, gold, 128 * W, torch.bfloat16, mag)
            if not r.ok:
                bad.append("it %d ar rank %d: %s" % (it, rank, r))
        else:
            o, gath = catcoc.allgather_matmul(a[:64], b)
            if ag_gold is None:
                ag_gold, _ = ref.allgather_matmul(a[:64], b, out_dtype=torch.float32)
            r = verify(o, ag_gold, 128, torch.bfloat16)
            if not r.ok:
                bad.append("it %d ag rank %d: %s" % (it, rank, r))
    ok = not bad
    for line in bad[:4]:
        print(line, flush=True)
    try:
        ctx.check("repeat")
    except RuntimeError as e:
        ok = False
        print("rank", rank, e, flush=True)
    report(name, ok)


class _DeviceCheck:
    """Acceptance rule of ``verify`` evaluated on the device and accumulated without a host
    synchronisation, so that the launches under test stay back to back."""

    def __init__(self, gold, k, dtype, magnitude=None):
        from mm_rs_with_catlass_b200.utils.verify import get_rtol
        g = gold.float()
        scale = g.abs() if magnitude is None else torch.maximum(g.abs(), magnitude.float())
        self.gold = g
        self.tol = get_rtol(dtype, k) * torch.clamp(scale, min=1.0)
        self.bad = torch.zeros((), dtype=torch.int64, device=gold.device)
        self.calls = 0

    def add(self, out):
        o = out.float()
        self.bad += ((o - self.gold).abs() > self.tol).sum() + (~torch.isfinite(o)).sum()
        self.calls += 1


def run_mixed_geometries(ctx, W, iters, name):
    """Back-to-back launches that alternate DIFFERENT tile geometries and ops on one context,
    several tiles per segment, rank-dependent data, no host synchronisation between calls and
    rank-dependent stalls in between (so ranks really run a launch apart). Every result of every
    iteration is checked on the device. This is the case in which stamp words or slab bytes
    shared between geometries would be overwritten by a rank that runs ahead or lags behind."""
    T = catcoc.TilingConfig
    bf = torch.bfloat16
    cases = []
    # reduce-scatter on 256-row pair tiles, 4 x 2 tiles per segment
    a, b = matmul_inputs(1024 * W, 512, 256, rank, bf, dev, seed=201)
    gold = ref.matmul_allreduce(a, b, out_dtype=torch.float32)
    mag = pmag(a, b)
    sl = slice(rank * 1024, (rank + 1) * 1024)
    t_rs_pair = T(bn=256, cta_pair=2, swizzle=2, pull=1)
    cases.append(("rs_pair", lambda a=a, b=b: catcoc.matmul_reduce_scatter(a, b, tiling=t_rs_pair),
                  _DeviceCheck(gold[sl], 256 * W, bf, mag[sl])))
    # all-reduce with column ownership on 128-row tiles (2 x 2 tiles per segment)
    a2, b2 = matmul_inputs(256, 256 * W, 192, rank, bf, dev, seed=202)
    gold2 = ref.matmul_allreduce(a2, b2, out_dtype=torch.float32)
    t_ar_cols = T(bn=128, seg_dim=1, use_multicast=bool(ctx.multicast))
    cases.append(("ar_cols", lambda: catcoc.matmul_allreduce(a2, b2, tiling=t_ar_cols).clone(),
                  _DeviceCheck(gold2, 192 * W, bf, pmag(a2, b2))))
    # all-gather with another K
    a3, b3 = matmul_inputs(192, 384, 320, rank, bf, dev, seed=203)
    gold3, _ = ref.allgather_matmul(a3, b3, out_dtype=torch.float32)
    cases.append(("ag", lambda: catcoc.allgather_matmul(a3, b3)[0], _DeviceCheck(gold3, 320, bf)))
    t_ag_mc = T(bn=128, use_multicast=True, comm_warps=3)
    cases.append(("ag_mc", lambda: catcoc.allgather_matmul(a3[:128], b3, tiling=t_ag_mc)[0],
                  _DeviceCheck(ref.allgather_matmul(a3[:128], b3, out_dtype=torch.float32)[0], 320, bf)))
    # quantised reduce-scatter on pair tiles with four lagged rounds
    x1, x2, s1, s2, bias = quant_inputs(1024 * W, 256, 256, rank, dev, seed=204)
    gold4 = ref.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias, out_dtype=torch.float32)
    t_q = T(bn=256, cta_pair=2, rounds=4)
    cases.append(("qrs_rounds4", lambda: catcoc.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias, tiling=t_q),
                  _DeviceCheck(gold4, 512, bf)))
    # reduce-scatter of another shape on single 128-column tiles, and an all-reduce by rows
    a5, b5 = matmul_inputs(256 * W, 384, 128, rank, bf, dev, seed=205)
    gold5 = ref.matmul_allreduce(a5, b5, out_dtype=torch.float32)
    mag5 = pmag(a5, b5)
    sl5 = slice(rank * 256, (rank + 1) * 256)
    t_single = T(bn=128, cta_pair=1, pull=0)
    cases.append(("rs_single", lambda: catcoc.matmul_reduce_scatter(a5, b5, tiling=t_single),
                  _DeviceCheck(gold5[sl5], 128 * W, bf, mag5[sl5])))
    t_ar_rows = T(bn=128, seg_dim=0, pull=0)
    cases.append(("ar_rows", lambda: catcoc.matmul_allreduce(a5, b5, tiling=t_ar_rows).clone(),
                  _DeviceCheck(gold5, 128 * W, bf, mag5)))
    # few rows and a long K: the split-K product + one-shot all-reduce path (its own buffer halves and stamps, the
    # same epoch counter as the fused kernels)
    a6, b6 = matmul_inputs(128, 1024, 2048, rank, bf, dev, seed=206)
    gold6 = ref.matmul_allreduce(a6, b6, out_dtype=torch.float32)
    cases.append(("ar_small", lambda: catcoc.matmul_allreduce(a6, b6), _DeviceCheck(gold6, 2048 * W, bf, pmag(a6, b6))))
    catcoc.matmul_allreduce(a6, b6)
    assert ctx.last_call.get("path", "").startswith("split-K"), ctx.last_call
    sl6 = slice(rank * (128 // W), (rank + 1) * (128 // W))
    cases.append(("rs_small", lambda: catcoc.matmul_reduce_scatter(a6, b6),
                  _DeviceCheck(gold6[sl6], 2048 * W, bf, pmag(a6, b6)[sl6])))
    # few rows in an all-gather GEMM: gather kernel + split-K product + plane reduction
    a7, b7 = matmul_inputs(64 // W if W <= 4 else 8, 512, 4096, rank, bf, dev, seed=207)
    gold7, ggold7 = ref.allgather_matmul(a7, b7, out_dtype=torch.float32)
    cases.append(("ag_small", lambda: catcoc.allgather_matmul(a7, b7)[0], _DeviceCheck(gold7, 4096, bf)))
    _, gath7 = catcoc.allgather_matmul(a7, b7)
    assert ctx.last_call.get("path", "").startswith("gather kernel"), ctx.last_call
    assert torch.equal(gath7, ggold7.to(bf)), "gathered activation of the small all-gather path"
    # the all-reduce result lives in the heap: the next call of another shape must not touch it
    keep = catcoc.matmul_allreduce(a2, b2, tiling=t_ar_cols)
    catcoc.matmul_allreduce(a5, b5, tiling=t_ar_rows)
    cases[1][2].add(keep)
    g = torch.Generator()
    g.manual_seed(4242)
    order = torch.randint(0, len(cases), (iters,), generator=g).tolist()
    stalls = torch.randint(0, W * 4, (iters,), generator=g).tolist()
    for it in range(iters):
        if stalls[it] == rank:
            torch.cuda._sleep(400000)   # about 0.2 ms: lets the other ranks run ahead
        _, fn, chk = cases[order[it]]
        chk.add(fn())
    ok = True
    try:
        ctx.check(name)
    except RuntimeError as e:
        ok = False
        print("rank", rank, e, flush=True)
    for cname, _, chk in cases:
        nbad = int(chk.bad.item())
        if nbad:
            ok = False
            print("rank %d: %s: %d elements out of tolerance over %d calls" % (rank, cname, nbad, chk.calls), flush=True)
    report(name, ok)


# default (pull flavour and multicast where the heap has the alias), push flavour, 2-CTA tiles, and the
# pull / multicast paths with few communication warps
TILINGS = [None, catcoc.TilingConfig(bn=128, cta_pair=1, pull=0), catcoc.TilingConfig(bn=256, cta_pair=2, swizzle=4),
           catcoc.TilingConfig(bn=128, pull=1, use_multicast=True, comm_warps=2)]

if mode == "ops":
    ctx = catcoc.init(heap_bytes=2 << 30, multicast=(os.environ.get("CATCOC_TEST_NVLS", "1") == "1"))
    W = world
    for dtype in (torch.bfloat16, torch.float16):
        for (M, N, K, ta, tb) in [(256 * W, 512, 384, False, False), (128 * W, 768, 256, False, True),
                                  (256 * W, 512, 320, True, False), (2 * W * 23, 328, 136, False, False),
                                  (W * 7, 72, 40, True, True)]:
            for ti, tiling in enumerate(TILINGS):
                a, b = matmul_inputs(M, N, K, rank, dtype, dev, trans_a=ta, trans_b=tb, seed=M + N)
                gold_full = ref.matmul_allreduce(a, b, trans_a=ta, trans_b=tb, out_dtype=torch.float32)
                mag = pmag(a, b, trans_a=ta, trans_b=tb)
                rows = M // W
                sl = slice(rank * rows, (rank + 1) * rows)
                tag = "%s_%dx%dx%d_%d%d_t%d" % (str(dtype)[6:], M, N, K, ta, tb, ti)
                # partial tiles cross the link rounded to the operand dtype: error scales with sum |partial|
                o = catcoc.matmul_reduce_scatter(a, b, trans_a=ta, trans_b=tb, tiling=tiling)
                check("rs_" + tag, o, gold_full[sl], K * W, dtype, mag[sl])
                o = catcoc.matmul_allreduce(a, b, trans_a=ta, trans_b=tb, tiling=tiling)
                check("ar_" + tag, o, gold_full, K * W, dtype, mag)
                # fp32 partials: the plain element-wise rule holds
                t32 = (tiling or catcoc.TilingConfig()).with_(fp32_partials=True)
                o = catcoc.matmul_reduce_scatter(a, b, trans_a=ta, trans_b=tb, tiling=t32)
                check("rs32_" + tag, o, gold_full[sl], K * W, dtype)
                o = catcoc.matmul_allreduce(a, b, trans_a=ta, trans_b=tb, tiling=t32)
                check("ar32_" + tag, o, gold_full, K * W, dtype)
        # all-reduce with fewer rows than ranks * 128: ownership splits by columns
        a, b = matmul_inputs(96, 1024, 256, rank, dtype, dev, seed=11)
        gold = ref.matmul_allreduce(a, b, out_dtype=torch.float32)
        mag = pmag(a, b)
        check("ar_smallM_%s" % str(dtype)[6:], catcoc.matmul_allreduce(a, b), gold, 256 * W, dtype, mag)
        # few rows and a long K: split-K product + one-shot all-reduce (auto tiling only); an explicit tiling keeps the
        # fused kernel on the same shape
        for (M2, N2, K2, tb2) in [(128, 1024, 2048, False), (96, 520, 4096, True), (256, 2048, 3072, False), (1, 128, 8192, False)]:
            a, b = matmul_inputs(M2, N2, K2, rank, dtype, dev, trans_b=tb2, seed=M2 + K2)
            gold = ref.matmul_allreduce(a, b, trans_b=tb2, out_dtype=torch.float32)
            mag = pmag(a, b, trans_b=tb2)
            tag = "%s_%dx%dx%d_%d" % (str(dtype)[6:], M2, N2, K2, tb2)
            o = catcoc.matmul_allreduce(a, b, trans_b=tb2)
            small = ctx.last_call.get("path", "").startswith("split-K")
            check("ar_oneshot_" + tag, o, gold, K2 * W, dtype, mag)
            from mm_rs_with_catlass_b200.ops.fused import _SMALL_AR_MAX_M
            report("ar_oneshot_path_" + tag, small == (M2 <= _SMALL_AR_MAX_M), str(ctx.last_call))
            given = torch.empty_like(o)
            check("ar_oneshot_out_" + tag, catcoc.matmul_allreduce(a, b, trans_b=tb2, out=given), gold, K2 * W, dtype, mag)
            check("ar_fused_" + tag, catcoc.matmul_allreduce(a, b, trans_b=tb2, tiling=catcoc.TilingConfig(bn=128)), gold,
                  K2 * W, dtype, mag)
            if M2 % W == 0:
                rws = M2 // W
                sl2 = slice(rank * rws, (rank + 1) * rws)
                o = catcoc.matmul_reduce_scatter(a, b, trans_b=tb2)
                from mm_rs_with_catlass_b200.ops.fused import _small_reduce_scatter_wanted
                report("rs_oneshot_path_" + tag, ctx.last_call.get("path", "").endswith("reduce-scatter")
                       == _small_reduce_scatter_wanted(M2, N2, K2, a.element_size(), W), str(ctx.last_call))
                check("rs_oneshot_" + tag, o, gold[sl2], K2 * W, dtype, mag[sl2])
                check("rs_oneshot_again_" + tag, catcoc.matmul_reduce_scatter(a, b, trans_b=tb2), gold[sl2], K2 * W, dtype, mag[sl2])
        # few rows in an all-gather GEMM: gather kernel + split-K product (auto tiling), fused kernel with a tiling
        for (m3, N3, K3, tb3) in [(16, 1024, 4096, False), (24, 520, 2048, True), (1, 256, 8192, False)]:
            a, b = matmul_inputs(m3, N3, K3, rank, dtype, dev, trans_b=tb3, seed=m3 + K3)
            gold, ggold = ref.allgather_matmul(a, b, trans_b=tb3, out_dtype=torch.float32)
            tag = "%s_%dx%dx%d_%d" % (str(dtype)[6:], m3, N3, K3, tb3)
            o, gath = catcoc.allgather_matmul(a, b, trans_b=tb3)
            report("ag_small_path_" + tag, ctx.last_call.get("path", "").startswith("gather kernel"), str(ctx.last_call))
            check("ag_small_" + tag, o, gold, K3, dtype)
            report("ag_small_gathered_" + tag, bool(torch.equal(gath, ggold.to(dtype))))
            o, gath = catcoc.allgather_matmul(a, b, trans_b=tb3)            # planned call, other buffer half
            check("ag_small_again_" + tag, o, gold, K3, dtype)
            report("ag_small_gathered_again_" + tag, bool(torch.equal(gath, ggold.to(dtype))))
            o, _ = catcoc.allgather_matmul(a, b, trans_b=tb3, tiling=catcoc.TilingConfig(bn=128))
            check("ag_fused_" + tag, o, gold, K3, dtype)
        a, b = matmul_inputs(96, 1024, 256, rank, dtype, dev, seed=11)
        gold = ref.matmul_allreduce(a, b, out_dtype=torch.float32)
        mag = pmag(a, b)
        for seg in (0, 1):
            check("ar_seg%d_%s" % (seg, str(dtype)[6:]),
                  catcoc.matmul_allreduce(a, b, tiling=catcoc.TilingConfig(bn=64, seg_dim=seg)), gold, 256 * W, dtype,
                  mag)
        # column ownership whose segments start inside a 128-byte column block of B (32 and 96
        # columns per rank): the block-wise 3-D fetch of an N-contiguous B cannot address them
        for cols, tb in ((32, False), (96, False), (96, True), (40, False)):
            a, b = matmul_inputs(256, cols * W, 192, rank, dtype, dev, trans_b=tb, seed=cols)
            gold = ref.matmul_allreduce(a, b, trans_b=tb, out_dtype=torch.float32)
            mag = pmag(a, b, trans_b=tb)
            for bn in (64, 128):
                check("ar_segcols%d_%d_bn%d_%s" % (cols, tb, bn, str(dtype)[6:]),
                      catcoc.matmul_allreduce(a, b, trans_b=tb, tiling=catcoc.TilingConfig(bn=bn, seg_dim=1)), gold,
                      192 * W, dtype, mag)
        # row ownership with an A stored [K, M] whose segments start inside a 128-byte block of A
        a, b = matmul_inputs(96 * W, 256, 192, rank, dtype, dev, trans_a=True, seed=5)
        gold = ref.matmul_allreduce(a, b, trans_a=True, out_dtype=torch.float32)
        mag = pmag(a, b, trans_a=True)
        check("rs_transA_seg96_%s" % str(dtype)[6:], catcoc.matmul_reduce_scatter(a, b, trans_a=True),
              gold[rank * 96:(rank + 1) * 96], 192 * W, dtype, mag[rank * 96:(rank + 1) * 96])
        check("ar_transA_seg96_%s" % str(dtype)[6:],
              catcoc.matmul_allreduce(a, b, trans_a=True, tiling=catcoc.TilingConfig(seg_dim=0)), gold, 192 * W, dtype, mag)
        if ctx.multicast:
            a, b = matmul_inputs(256 * W, 512, 256, rank, dtype, dev, seed=12)
            gold = ref.matmul_allreduce(a, b, out_dtype=torch.float32)
            check("ar_nvls_%s" % str(dtype)[6:],
                  catcoc.matmul_allreduce(a, b, tiling=catcoc.TilingConfig(use_multicast=True)), gold, 256 * W, dtype,
                  pmag(a, b))
        for (m, N, K, tb) in [(256, 512, 512, False), (384, 640, 1024, True), (100, 328, 136, False), (64, 256, 6148, False)]:
            for ti, tiling in enumerate(TILINGS):
                a, b = matmul_inputs(m, N, K, rank, dtype, dev, trans_b=tb, seed=m + K)
                gold, gath = ref.allgather_matmul(a, b, trans_b=tb, out_dtype=torch.float32)
                o, g = catcoc.allgather_matmul(a, b, trans_b=tb, tiling=tiling)
                tag = "%s_%dx%dx%d_%d_t%d" % (str(dtype)[6:], m, N, K, tb, ti)
                check("ag_" + tag, o, gold, K, dtype)
                report("ag_gathered_" + tag, bool(torch.equal(g, gath)))
    # all-gather GEMM with the activation in its epilogue (shard by multicast and by peer stores)
    from mm_rs_with_catlass_b200.ops._common import apply_activation
    for act, mc in (("gelu", True), ("silu", False)):
        a, b = matmul_inputs(200, 392, 264, rank, torch.bfloat16, dev, seed=71, b_std=0.2)
        gold, _ = ref.allgather_matmul(a, b, out_dtype=torch.float32)
        o, _ = catcoc.allgather_matmul(a, b, activation=act, tiling=catcoc.TilingConfig(bn=128, use_multicast=mc))
        check("ag_%s_mc%d" % (act, mc), o, apply_activation(gold, act), 264, torch.bfloat16)
    for (M, N, K, tb, with_bias) in [(128 * W, 512, 512, False, True), (256 * W, 768, 384, True, True),
                                     (4 * W, 512, 128, False, False), (W * 23, 136, 72, True, True)]:
        for out_dtype in (torch.bfloat16, torch.float16):
            x1, x2, s1, s2, bias = quant_inputs(M, N, K, rank, dev, trans_b=tb, with_bias=with_bias, seed=K)
            gold = ref.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias, trans_b=tb, out_dtype=torch.float32)
            o = catcoc.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias, trans_b=tb, out_dtype=out_dtype)
            check("qrs_%dx%dx%d_%d_%s" % (M, N, K, tb, str(out_dtype)[6:]), o, gold, 512, out_dtype)
    # block-scaled fp8 (mxf8) row-parallel linear with the fused reduce-scatter
    if hasattr(torch, "float8_e4m3fn"):
        for (M, N, K) in [(256 * W, 384, 512), (128 * W, 256, 1024), (128 * W, 136, 96)]:
            g = torch.Generator(device=dev)
            g.manual_seed(900 + rank)
            a = torch.randn(M, K, device=dev, generator=g)
            b = torch.randn(N, K, device=dev, generator=g) * 0.1
            a = a * torch.exp2(torch.randint(-3, 3, (M, K // 32), device=dev, generator=g).float()).repeat_interleave(32, 1)
            aq, sa = catcoc.quantize_mxf8(a)
            bq, sb = catcoc.quantize_mxf8(b)
            full = catcoc.dequantize_mxf8(aq, sa) @ catcoc.dequantize_mxf8(bq, sb).t()
            mag = full.abs()
            dist.all_reduce(full)
            dist.all_reduce(mag)
            rows = M // W
            sl = slice(rank * rows, (rank + 1) * rows)
            o = catcoc.mxf8_matmul_reduce_scatter(aq, catcoc.pack_scales(sa), bq, catcoc.pack_scales(sb))
            check("mxf8_rs_%dx%dx%d" % (M, N, K), o, full[sl], K * W, torch.bfloat16, mag[sl])
            o = catcoc.mxf8_matmul_reduce_scatter(aq, catcoc.pack_scales(sa), bq, catcoc.pack_scales(sb),
                                                  tiling=catcoc.TilingConfig(fp32_partials=True))
            check("mxf8_rs32_%dx%dx%d" % (M, N, K), o, full[sl], K * W, torch.bfloat16)
    # debug pattern (all-ones operands, arange bias) localises indexing errors
    x1, x2, s1, s2, bias = quant_inputs(32 * W, 256, 128, rank, dev, debug=True)
    o = catcoc.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias, out_dtype=torch.float32)
    exp = ((128.0 + torch.arange(1, 257, device=dev).float()) * W * 1e-4)[None, :].expand(32, 256)
    report("qrs_debug_pattern", bool(torch.allclose(o, exp, rtol=1e-5)))
    run_mixed_launches(ctx, W, 60, "repeat_60_mixed_launches")
    run_mixed_geometries(ctx, W, 120, "mixed_geometries_120")
    # the flagship block
    from mm_rs_with_catlass_b200.models.tp_mlp import TPMLP, TPMLPConfig
    mlp = TPMLP(TPMLPConfig(hidden=512, ffn=256 * W), ctx, dev)
    x = torch.randn(128, 512, device=dev).bfloat16()
    h_ref, _ = ref.allgather_matmul(x, mlp.w_up, out_dtype=torch.bfloat16)
    check("tpmlp", mlp(x), mlp.reference_forward(x).float(), 256 * W, torch.bfloat16,
          pmag(mlp._act(h_ref), mlp.w_down)[rank * 128:(rank + 1) * 128])
    ctx.finalize()

elif mode == "repeat":
    # the mixed-launch loop alone, long: cheap to run when hunting a protocol race
    ctx = catcoc.init(heap_bytes=1 << 30, multicast=(os.environ.get("CATCOC_TEST_NVLS", "1") == "1"))
    run_mixed_launches(ctx, world, int(os.environ.get("CATCOC_TEST_REPEATS", "600")), "repeat_mixed_launches")
    ctx.finalize()

elif mode == "prims":
    # SHMEM primitives over peer memory and the multicast alias: put / get with a signal, multicast
    # broadcast, and the numerics of the in-switch sum that the pull flavours rely on
    ctx = catcoc.init(heap_bytes=256 << 20)
    n = 1 << 20
    g = torch.Generator(device=dev)
    g.manual_seed(31 + rank)
    x = (torch.randn(n, device=dev, generator=g) * (1.0 + rank)).to(torch.bfloat16)
    buf = ctx.malloc(2 * n)
    sig = ctx.malloc(256)
    sig.tensor(torch.int32).zero_()
    buf.tensor(torch.bfloat16, (n,)).copy_(x)
    ctx.barrier()
    # get: read the right neighbour's buffer; put: write mine into the left neighbour's scratch
    peer = (rank + 1) % world
    got = torch.empty(n, dtype=torch.bfloat16, device=dev)
    ctx.get(peer, got, buf)
    xs = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(xs, x)
    report("shmem_get_reads_the_peer", bool(torch.equal(got, xs[peer])))
    scratch = ctx.malloc(2 * n)
    ctx.put((rank - 1) % world, scratch, x, signal=sig, signal_value=1)
    ctx.wait_until(sig, ctx.put_blocks(), timeout_ms=2000.0)
    torch.cuda.synchronize()
    report("shmem_put_signal_wait", bool(torch.equal(scratch.tensor(torch.bfloat16, (n,)), xs[peer])))
    if ctx.multicast:
        exact = torch.stack([t.float() for t in xs]).sum(0)           # exact in fp32 for a handful of bf16 terms
        out = torch.empty(n, dtype=torch.bfloat16, device=dev)
        ctx.mc_reduce_bf16(out, buf)
        torch.cuda.synchronize()
        rn = exact.to(torch.bfloat16)
        rz = (exact.view(torch.int32) & -65536).view(torch.float32).to(torch.bfloat16)
        ulp = torch.exp2(torch.floor(torch.log2(exact.abs().clamp(min=1e-30))) - 7)
        err = (out.float() - exact).abs()
        within = bool((err <= ulp * 1.0001).all())
        frac_rn = float((out == rn).float().mean())
        frac_rz = float((out == rz).float().mean())
        if rank == 0:
            print(json.dumps({"case": "switch_sum_numerics", "ok": within, "equal_to_round_nearest": frac_rn,
                              "equal_to_truncation": frac_rz, "max_err_in_ulp": float((err / ulp).max())}), flush=True)
        report("switch_sum_within_one_ulp_of_the_exact_sum", within)
        dst = ctx.malloc(2 * n)
        ctx.barrier()
        if rank == 0:
            ctx.mc_broadcast(dst, x)
        ctx.barrier()
        torch.cuda.synchronize()
        report("multicast_broadcast_lands_everywhere", bool(torch.equal(dst.tensor(torch.bfloat16, (n,)), xs[0])))
    ctx.check("prims")
    ctx.finalize()

elif mode == "bench_shapes":
    # the shapes and tilings that ship: every fused op at the benchmark's LLM tensor-parallel shape (M = 8192,
    # hidden 8192, FFN 28672 / W) with the tiling the chooser picks, against an fp32 golden computed on the GPUs
    ctx = catcoc.init(heap_bytes=6 << 30)
    W, M, H, F = world, 8192, 8192, 28672
    kf = F // W
    bf = torch.bfloat16
    a, b = matmul_inputs(M, H, kf, rank, bf, dev, seed=1, b_std=0.02)
    gold = ref.matmul_allreduce(a, b, out_dtype=torch.float32)
    mag = pmag(a, b)
    rows = M // W
    sl = slice(rank * rows, (rank + 1) * rows)
    check("bench_rs", catcoc.matmul_reduce_scatter(a, b), gold[sl], F, bf, mag[sl])
    check("bench_ar", catcoc.matmul_allreduce(a, b), gold, F, bf, mag)
    for name, t in (("pull", catcoc.TilingConfig(bn=256, cta_pair=2, pull=1, use_multicast=True)),
                    ("push_tma", catcoc.TilingConfig(bn=256, cta_pair=2, pull=0, push_tma=1))):
        check("bench_rs_" + name, catcoc.matmul_reduce_scatter(a, b, tiling=t), gold[sl], F, bf, mag[sl])
        check("bench_ar_" + name, catcoc.matmul_allreduce(a, b, tiling=t), gold, F, bf, mag)
    del gold, mag
    x1, x2, s1, s2, bias = quant_inputs(M, H, kf, rank, dev, seed=3)
    goldq = ref.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias, out_dtype=torch.float32)
    check("bench_quant", catcoc.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias), goldq, 512, bf)
    del x1, x2, goldq, a, b
    torch.cuda.empty_cache()
    a, b = matmul_inputs(M // W, kf, H, rank, bf, dev, seed=2, b_std=0.02)
    golda, gath = ref.allgather_matmul(a, b, out_dtype=torch.float32)
    for name, t in (("default", None), ("multicast", catcoc.TilingConfig(bn=256, cta_pair=2, use_multicast=True)),
                    ("peer_stores", catcoc.TilingConfig(bn=256, cta_pair=2, use_multicast=False))):
        o, g = catcoc.allgather_matmul(a, b, tiling=t)
        check("bench_ag_" + name, o, golda, H, bf)
        report("bench_ag_gathered_" + name, bool(torch.equal(g, gath)))
    ctx.finalize()

elif mode == "checked":
    # the fused ops under the bounds-checked build of the library (CATCOC_CHECKED=1 in the environment):
    # pull and push flavours, both tile flavours, ragged shapes, all-gather by multicast and by peer stores
    from mm_rs_with_catlass_b200 import _native as N
    ctx = catcoc.init(heap_bytes=1 << 30)
    report("checked_build_loaded", N.lib().catcoc_is_checked_build() == 1)
    W = world
    T = catcoc.TilingConfig
    for (M, Nn, K) in [(256 * W, 512, 384), (2 * W * 23, 328, 136)]:
        a, b = matmul_inputs(M, Nn, K, rank, torch.bfloat16, dev, seed=M)
        gold = ref.matmul_allreduce(a, b, out_dtype=torch.float32)
        mag = pmag(a, b)
        rows = M // W
        sl = slice(rank * rows, (rank + 1) * rows)
        for ti, t in enumerate([T(bn=128, pull=0), T(bn=256, cta_pair=2, pull=1), T(bn=64, pull=1, comm_warps=1)]):
            check("chk_rs_%d_t%d" % (M, ti), catcoc.matmul_reduce_scatter(a, b, tiling=t), gold[sl], K * W,
                  torch.bfloat16, mag[sl])
            check("chk_ar_%d_t%d" % (M, ti), catcoc.matmul_allreduce(a, b, tiling=t), gold, K * W, torch.bfloat16, mag)
    for (m, Nn, K, mc) in [(256, 512, 512, True), (100, 328, 136, False), (64, 256, 6148, True)]:
        a, b = matmul_inputs(m, Nn, K, rank, torch.bfloat16, dev, seed=m + K)
        gold, gath = ref.allgather_matmul(a, b, out_dtype=torch.float32)
        o, g = catcoc.allgather_matmul(a, b, tiling=T(bn=128, use_multicast=mc))
        check("chk_ag_%dx%dx%d" % (m, Nn, K), o, gold, K, torch.bfloat16)
        report("chk_ag_gathered_%d" % m, bool(torch.equal(g, gath)))
    x1, x2, s1, s2, bias = quant_inputs(256 * W, 768, 384, rank, dev, seed=9)
    gold = ref.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias, out_dtype=torch.float32)
    check("chk_qrs", catcoc.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias, tiling=T(bn=256, cta_pair=2, rounds=2)),
          gold, 512, torch.bfloat16)
    ctx.finalize()

elif mode == "mixed":
    # different geometries back to back, no synchronisation between the calls
    ctx = catcoc.init(heap_bytes=2 << 30, multicast=(os.environ.get("CATCOC_TEST_NVLS", "1") == "1"))
    run_mixed_geometries(ctx, world, int(os.environ.get("CATCOC_TEST_REPEATS", "400")), "mixed_geometries")
    ctx.finalize()

elif mode == "withhold":
    # Failure detection without a GPU fault: the last rank posts no stamps, so its peers' waits
    # run out of their (short) budget, return an error status and raise on the host. NVLS off.
    from mm_rs_with_catlass_b200 import _native as N
    from mm_rs_with_catlass_b200.ops import fused
    os.environ["CATCOC_TIMEOUT_MS"] = "300"
    ctx = catcoc.init(heap_bytes=256 << 20, multicast=False)
    a, b = matmul_inputs(128 * world, 256, 128, rank, torch.bfloat16, dev)
    orig = fused.cm.launch

    def launch_withholding(args, device):
        # the argument block may be a cached launch plan: leave it as it was found
        if rank == world - 1:
            args.withhold_signals = 1
        try:
            return orig(args, device)
        finally:
            args.withhold_signals = 0

    fused.cm.launch = launch_withholding
    catcoc.matmul_reduce_scatter(a, b)
    torch.cuda.synchronize()
    raised = False
    try:
        ctx.check("withheld signal")
    except RuntimeError as e:
        raised = "never arrived" in str(e)
    fused.cm.launch = orig
    expect_raise = rank != world - 1 or world == 1
    # the withholding rank itself still receives everybody's tiles and finishes cleanly
    report("withheld_signal_detected", raised == expect_raise)
    ctx.reset_after_error()
    gold = ref.matmul_reduce_scatter(a, b, out_dtype=torch.float32)
    o = catcoc.matmul_reduce_scatter(a, b)
    rows = 128
    check("recovers_after_reset", o, gold, 128 * world, torch.bfloat16,
          pmag(a, b)[rank * rows:(rank + 1) * rows])
    ctx.finalize()

dist.barrier()
dist.destroy_process_group()
sys.exit(1 if failures else 0)
