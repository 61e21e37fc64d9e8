"""TilingConfig, the search space and its feasibility rules, the measured table and the chooser."""
import math

import pytest
import torch

from mm_rs_with_catlass_b200.tiling import chooser, search
from mm_rs_with_catlass_b200.tiling.config import TilingConfig
from mm_rs_with_catlass_b200.tiling.table import COLUMNS, Row, TilingTable


def test_config_validation():
    TilingConfig(bn=128, cta_pair=2).validate()
    for bad in (dict(bn=96), dict(cta_pair=3), dict(bn=64, cta_pair=2), dict(seg_dim=2), dict(num_ctas=-1)):
        with pytest.raises(ValueError):
            TilingConfig(**bad).validate()
    assert TilingConfig().effective_bn == 256
    assert set(["m0", "n0", "k0", "comm_interval", "comm_tile_m", "comm_block_m", "comm_npu_split",
                "comm_data_split"]) <= set(TilingConfig().to_dict())      # the reference's CocTilingParams fields


def test_candidates_respect_the_rules():
    p = search.Problem("matmul_reduce_scatter", 8192, 8192, 3584, 8)
    cands = search.candidates(p)
    assert cands and all(search.infeasible_reason(p, t) is None for t in cands)
    assert all(t.seg_dim == -1 and not t.use_multicast for t in cands)
    assert not any(t.cta_pair == 2 and t.effective_bn == 64 for t in cands)
    q = search.Problem("quant_matmul_reduce_scatter", 8192, 8192, 3584, 8, dtype="int8")
    assert all((t.effective_bn // (2 if t.cta_pair == 2 else 1)) >= 128 for t in search.candidates(q))
    ar = search.Problem("matmul_allreduce", 128, 8192, 3584, 8, multicast_available=True)
    assert {t.seg_dim for t in search.candidates(ar)} == {0, 1}
    assert any(t.use_multicast for t in search.candidates(ar))


def test_infeasible_reasons():
    rs = search.Problem("matmul_reduce_scatter", 1001, 512, 256, 8)
    assert "divide" in search.infeasible_reason(rs, TilingConfig())
    ag = search.Problem("allgather_matmul", 1024, 512, 256, 2, trans_a=True)
    assert "trans_a" in search.infeasible_reason(ag, TilingConfig())
    ar = search.Problem("matmul_allreduce", 128, 8 * 1001, 256, 8)
    assert "aligned" in search.infeasible_reason(ar, TilingConfig(seg_dim=1))
    small = search.Problem("matmul_allreduce", 16384, 8192, 3584, 8, heap_bytes=64 << 20)
    assert "heap" in search.infeasible_reason(small, TilingConfig(seg_dim=0))
    nomc = search.Problem("matmul_allreduce", 1024, 1024, 256, 2)
    assert "multicast" in search.infeasible_reason(nomc, TilingConfig(use_multicast=True))
    assert "multicast alias" in search.infeasible_reason(nomc, TilingConfig(pull=1))
    q = search.Problem("quant_matmul_reduce_scatter", 1024, 1024, 256, 8, dtype="int8", multicast_available=True)
    assert "16-bit" in search.infeasible_reason(q, TilingConfig(pull=1))
    odd = search.Problem("matmul_reduce_scatter", 1024, 1004, 256, 4, multicast_available=True)
    assert "multiples of 8" in search.infeasible_reason(odd, TilingConfig(pull=1))


def test_workspace_estimate_matches_hand_count():
    p = search.Problem("matmul_reduce_scatter", 8192, 8192, 3584, 8)
    t = TilingConfig(bn=256, cta_pair=1)
    tiles_per_seg = (1024 // 128) * (8192 // 256)
    assert search.workspace_bytes(p, t) == 2 * 8 * tiles_per_seg * 128 * 256 * 2 + 4 * tiles_per_seg * 8 * 4
    assert search.workspace_bytes(search.Problem("matmul", 1, 1, 1, 1), t) == 0


def _row(op, m, k, n, us, **kw):
    return Row(op, m, k, n, 0, 0, "bf16", 8, TilingConfig(**kw), us)


def test_table_roundtrip_best_and_resume(tmp_path):
    path = tmp_path / "t.csv"
    rows = [_row("matmul_reduce_scatter", 8192, 3584, 8192, 410.0, bn=256, cta_pair=1),
            _row("matmul_reduce_scatter", 8192, 3584, 8192, 380.0, bn=256, cta_pair=2),
            _row("matmul_reduce_scatter", 1024, 3584, 8192, 70.0, bn=128)]
    for r in rows:
        assert TilingTable.append_row(path, r)
    assert not TilingTable.append_row(path, rows[0])            # resumable: duplicates are skipped
    head = path.read_text().splitlines()[0].split(",")
    assert head == COLUMNS and head[:12] == ["Op", "M", "K", "N", "Transpose A", "Transpose B", "commInterval",
                                             "commTileM", "commBlockM", "commNpuSplit", "commDataSplit", "Time(us)"]
    tbl = TilingTable.load(path)
    assert len(tbl.rows) == 3
    best = tbl.best()
    assert len(best.rows) == 2
    assert best.lookup("matmul_reduce_scatter", 8192, 8192, 3584, 8, torch.bfloat16).cta_pair == 2
    # nearest shape within a factor of two, nothing beyond
    assert best.lookup("matmul_reduce_scatter", 6000, 8192, 3584, 8, torch.bfloat16).cta_pair == 2
    assert best.lookup("matmul_reduce_scatter", 64, 8192, 3584, 8, torch.bfloat16) is None
    assert best.lookup("matmul_allreduce", 8192, 8192, 3584, 8, torch.bfloat16) is None
    best.save(tmp_path / "best.csv")
    assert len(TilingTable.load(tmp_path / "best.csv").rows) == 2


def test_heuristic_follows_the_cost_model_and_is_deterministic():
    big = chooser.heuristic("matmul_reduce_scatter", 8192, 8192, 3584, 8, torch.bfloat16)
    assert big.effective_bn == 256 and big.cta_pair == 2
    # one row of tiles: only narrow tiles give every SM something to do
    small = chooser.heuristic("matmul_allreduce", 128, 8192, 3584, 8, torch.bfloat16)
    assert small.effective_bn == 64 and small.cta_pair == 1
    assert math.ceil(128 / 128) * (8192 // small.effective_bn) >= 128
    assert chooser.heuristic("matmul", 128, 8192, 1024, 1, torch.bfloat16).effective_bn == 64
    # from a few hundred rows on the widest tile wins although it leaves SMs idle (measured)
    for m, n in ((512, 8192), (1024, 4096), (2048, 2048)):
        mid = chooser.heuristic("matmul", m, n, 4096, 1, torch.bfloat16)
        assert mid.effective_bn == 256 and mid.cta_pair == 2
    assert chooser.tile_cost(1024, 1, 4096, 256, 2) < chooser.tile_cost(1024, 1, 4096, 128, 2)
    assert chooser.tile_cost(128, 1, 8192, 64, 1) < chooser.tile_cost(128, 1, 8192, 256, 1)
    q = chooser.heuristic("quant_matmul_reduce_scatter", 256, 512, 512, 2, torch.int8)
    assert q.effective_bn >= 128
    assert chooser.heuristic("matmul_reduce_scatter", 8192, 8192, 3584, 8, torch.bfloat16) == big
    tbl = TilingTable([_row("matmul_reduce_scatter", 8192, 3584, 8192, 1.0, bn=128, swizzle=4)])
    assert chooser.choose("matmul_reduce_scatter", 8192, 8192, 3584, 8, torch.bfloat16, table=tbl).bn == 128


def test_mx_scale_packing_matches_the_tensor_core_block_layout():
    from mm_rs_with_catlass_b200.ops import mx
    x = torch.randn(200, 160) * torch.exp2(torch.randint(-6, 6, (200, 5)).float()).repeat_interleave(32, 1)
    q, s = mx.quantize_mxf8(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (200, 5) and s.dtype == torch.uint8
    d = mx.dequantize_mxf8(q, s)
    assert (d - x).abs().max() <= 2 ** -3 * x.abs().max()          # e4m3: 3 mantissa bits
    assert q.float().abs().max() <= 448.0
    p = mx.pack_scales(s)
    assert p.shape == (2, 2, 512)
    for r, kb in ((0, 0), (31, 4), (32, 1), (137, 3), (199, 2)):
        assert int(p[r // 128, kb // 4, (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4]) == int(s[r, kb])
    assert int(p[1, 1, (10 % 32) * 16 + 3 * 4 + 3]) == 127          # padding is the neutral scale
    with pytest.raises(ValueError):
        mx.quantize_mxf8(torch.randn(4, 40))


def test_search_space_offers_both_data_paths_where_the_heap_has_a_multicast_alias():
    rs = search.Problem("matmul_reduce_scatter", 8192, 8192, 3584, 8, multicast_available=True)
    cands = search.candidates(rs)
    assert {t.pull for t in cands} == {0, 1}
    assert all(t.rounds == 0 for t in cands if t.pull == 1)
    ag = search.Problem("allgather_matmul", 8192, 3584, 8192, 8, multicast_available=True)
    assert {t.use_multicast for t in search.candidates(ag)} == {False, True}
    ar = search.Problem("matmul_allreduce", 8192, 8192, 3584, 8, multicast_available=True)
    assert all(t.use_multicast for t in search.candidates(ar) if t.pull == 1)
    # without the alias only the push flavour and peer stores remain
    rs_p2p = search.Problem("matmul_reduce_scatter", 8192, 8192, 3584, 8)
    assert {t.pull for t in search.candidates(rs_p2p)} == {0}
    assert len(set(cands)) == len(cands)


def test_shipped_table_covers_every_benchmark_configuration():
    """Every LLM tensor-parallel configuration of the benchmark (hidden 8192, FFN 28672, sharded over 2, 4 and
    8 GPUs) resolves to a measured row: an exact hit or a neighbour within a factor of two per dimension."""
    import torch
    from mm_rs_with_catlass_b200.tiling import table
    tbl = table.TilingTable.load(table.DEFAULT_TABLE_PATH).best()
    H, F = 8192, 28672
    ops = {"matmul_allreduce": (128, 1024, 8192), "allgather_matmul": (1024, 8192, 16384),
           "matmul_reduce_scatter": (1024, 8192, 16384), "quant_matmul_reduce_scatter": (128, 1024, 8192, 16384)}
    missing = []
    for W in (2, 4, 8):
        for op, Ms in ops.items():
            for M in Ms:
                m, n, k = (M, F // W, H) if op == "allgather_matmul" else (M, H, F // W)
                dt = torch.int8 if op.startswith("quant") else torch.bfloat16
                if tbl.lookup(op, m, n, k, W, dt) is None:
                    missing.append((W, op, M))
    assert not missing, missing
