"""The bounds-checked build of the library (``CATCOC_CHECKED=1``): every workspace, peer, output
and accumulator offset of the kernels is compared with the extent of its buffer; an offset
outside is recorded in the status block (site, limit, offset) and the access is skipped. The
tests run it in child processes (the build is chosen when the library is loaded): the small-case
matrix must pass under it without a report, and an output whose extent is understated (the
buffer itself is large enough, so nothing is ever written out of bounds) must be reported with
its site and left untouched beyond the stated extent."""
import json
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _child(code: str, env_extra=None, timeout=600):
    env = dict(os.environ, CATCOC_CHECKED="1", PYTHONPATH=REPO)
    env.update(env_extra or {})
    proc = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], capture_output=True, text=True, env=env,
                          timeout=timeout, cwd=REPO)
    assert proc.returncode == 0, "child failed:\n%s\n%s" % (proc.stdout[-3000:], proc.stderr[-3000:])
    return [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]


def test_local_kernels_pass_under_the_checked_build():
    out = _child("""
        import json, torch
        import mm_rs_with_catlass_b200 as catcoc
        from mm_rs_with_catlass_b200 import _native as N
        from mm_rs_with_catlass_b200.ops._common import local_status, raise_on_status
        from mm_rs_with_catlass_b200.utils.verify import assert_close
        assert N.lib().catcoc_is_checked_build() == 1
        dev = torch.device("cuda:0")
        for (m, n, k, pair, bn) in [(256, 512, 384, 1, 256), (23, 45, 68 + 4, 1, 64), (1000, 328, 136, 1, 128),
                                    (512, 512, 256, 2, 256), (300, 200, 264, 2, 128)]:
            a = torch.randn(m, k, device=dev).bfloat16()
            b = (torch.randn(k, n, device=dev) * 0.1).bfloat16()
            o = catcoc.matmul(a, b, tiling=catcoc.TilingConfig(bn=bn, cta_pair=pair))
            assert_close(o, a.float() @ b.float(), k=k, dtype=torch.bfloat16, what="%dx%dx%d" % (m, n, k))
        x1 = torch.randint(-127, 128, (200, 256), device=dev, dtype=torch.int32).to(torch.int8)
        x2 = torch.randint(-127, 128, (256, 384), device=dev, dtype=torch.int32).to(torch.int8)
        o = catcoc.matmul(x1, x2)
        assert torch.equal(o.cpu().long(), x1.cpu().long() @ x2.cpu().long())
        torch.cuda.synchronize()
        raise_on_status(local_status(dev), "checked build")
        print(json.dumps({"ok": True}))
    """)
    assert out and out[-1]["ok"]


def test_an_understated_output_extent_is_reported_and_nothing_is_written_past_it():
    out = _child("""
        import ctypes as C, json, torch
        import mm_rs_with_catlass_b200 as catcoc
        from mm_rs_with_catlass_b200 import _native as N
        from mm_rs_with_catlass_b200.ops import _common as cm
        dev = torch.device("cuda:0")
        m, n, k = 256, 256, 128
        a = torch.randn(m, k, device=dev).bfloat16()
        b = torch.randn(k, n, device=dev).bfloat16()
        out = torch.full((m, n), 7.0, device=dev, dtype=torch.bfloat16)
        status = torch.zeros(8, dtype=torch.int32, device=dev)
        args = N.OpArgs()
        args.mode, args.in_fmt = N.MODE_LOCAL, N.IN_BF16
        args.M, args.N, args.K = m, n, k
        args.a, args.lda, args.b, args.ldb = a.data_ptr(), k, b.data_ptr(), n
        args.out, args.ldc, args.out_fmt, args.partial_fmt = out.data_ptr(), n, N.FMT_BF16, N.FMT_BF16
        args.tiling.bn = 128
        args.rank, args.W = 0, 1
        args.status = status.data_ptr()
        args.limit[N.LIM_OUT] = 128 * n * 2            # the caller claims half of the rows
        cm.launch(args, dev)
        torch.cuda.synchronize()
        st = status.cpu().tolist()
        print(json.dumps({"status": st, "tail_untouched": bool((out[128:] == 7.0).all().item()),
                          "head_written": bool((out[:128] != 7.0).any().item())}))
    """, {"CATCOC_OUT_TMA": "0"})
    r = out[-1]
    assert r["status"][0] == 7, r            # STATUS_OUT_OF_RANGE
    assert r["status"][2] == 13, r           # SITE_OUT_STORE
    assert r["status"][3] == 128 * 256 * 2, r
    assert r["tail_untouched"] and r["head_written"], r


def test_the_launcher_refuses_a_tensor_map_over_an_understated_output():
    out = _child("""
        import json, torch
        from mm_rs_with_catlass_b200 import _native as N
        from mm_rs_with_catlass_b200.ops import _common as cm
        dev = torch.device("cuda:0")
        m, n, k = 256, 256, 128
        a = torch.randn(m, k, device=dev).bfloat16(); b = torch.randn(k, n, device=dev).bfloat16()
        out = torch.empty((m, n), device=dev, dtype=torch.bfloat16)
        status = torch.zeros(8, dtype=torch.int32, device=dev)
        args = N.OpArgs()
        args.mode, args.in_fmt = N.MODE_LOCAL, N.IN_BF16
        args.M, args.N, args.K = m, n, k
        args.a, args.lda, args.b, args.ldb = a.data_ptr(), k, b.data_ptr(), n
        args.out, args.ldc, args.out_fmt, args.partial_fmt = out.data_ptr(), n, N.FMT_BF16, N.FMT_BF16
        args.rank, args.W = 0, 1
        args.status = status.data_ptr()
        args.limit[N.LIM_OUT] = 100
        try:
            cm.launch(args, dev)
            print(json.dumps({"refused": False}))
        except N.NativeError as e:
            print(json.dumps({"refused": True, "code": e.code, "msg": str(e)}))
    """)
    assert out[-1]["refused"] and out[-1]["code"] == -1 and "smaller than" in out[-1]["msg"]


def test_fused_ops_on_two_gpus_pass_under_the_checked_build(gpu_count):
    if gpu_count < 2:
        pytest.skip("needs 2 GPUs")
    from test_fused_multi_gpu import _run
    cases = _run(2, "checked", {"CATCOC_CHECKED": "1", "CATCOC_TIMEOUT_MS": "3000"}, timeout=600)
    assert len(cases) >= 12


def test_event_ring_gives_a_chrome_trace_with_matched_begin_and_end_records(tmp_path):
    path = str(tmp_path / "trace.json")
    out = _child("""
        import json, torch
        import mm_rs_with_catlass_b200 as catcoc
        from mm_rs_with_catlass_b200.utils.trace import EventTrace
        dev = torch.device("cuda:0")
        a = torch.randn(1024, 512, device=dev).bfloat16()
        b = torch.randn(512, 1024, device=dev).bfloat16()
        with EventTrace(capacity=4096) as tr:
            catcoc.matmul(a, b, tiling=catcoc.TilingConfig(bn=256, cta_pair=1))
        recs = tr.records()
        n = tr.dump_chrome(%r)
        by = {}
        for r in recs:
            by.setdefault((r["cta"], r["role"], r["tile"]), []).append(r["phase"])
        epi = [k for k in by if k[1] == 2]
        print(json.dumps({"events": n, "dropped": tr.dropped, "epilogue_tiles": len(epi),
                          "paired": all(sorted(by[k]) == [0, 1] for k in epi),
                          "ordered": all(x["t_ns"] <= y["t_ns"] for x, y in zip(recs, recs[1:]))}))
    """ % path)
    r = out[-1]
    assert r["epilogue_tiles"] == 32 and r["paired"] and r["ordered"] and r["dropped"] == 0, r   # 8 x 4 tiles
    with open(path) as fh:
        trace = json.load(fh)
    assert len([e for e in trace["traceEvents"] if e.get("ph") in ("B", "E")]) == r["events"]
