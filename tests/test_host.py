"""Host-side logic of libcutespmm that needs no GPU: the library loads and exports its header's
symbols, the plan builder's views agree with the reference's preprocessing (golden vectors), the
packed format round-trips, bad input is rejected with an error code, the loader matches MTX_READER."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

import cutespmm_ae_b200 as cs
from cutespmm_ae_b200 import generators as g
from conftest import GOLDEN, GOLDEN_CASES, ROOT, load_golden


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "cutespmm.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    names = set(re.findall(r"\b(cutespmm_[a-z0-9_]+)\s*\(", header))
    assert len(names) >= 18
    lib = ctypes.CDLL(str(cs._build.LIB))
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, missing
    assert cs.lib.cutespmm_version() >= 100


def test_status_strings():
    assert cs.lib.cutespmm_status_string(0) == b"success"
    assert b"invalid" in cs.lib.cutespmm_status_string(-1)


@pytest.mark.parametrize("name", [c for c in GOLDEN_CASES if c != "uniform_256_unsorted"])
def test_panel_views_match_reference_preprocessing(name):
    gd = load_golden(name)
    p = cs.Plan(int(gd["M"]), int(gd["K"]), gd["row_ptr"], gd["cols"], gd["vals"], host_only=True)
    assert np.array_equal(p.blocked_row_ptr(), gd["blocked_row_ptr"])
    assert np.array_equal(p.active_cols(), gd["active_cols"])
    info = p.info()
    assert info["num_panels"] == int(gd["M"]) // 16
    assert info["nnz"] == gd["cols"].size


@pytest.mark.parametrize("path", [cs.PATH_ROWS, cs.PATH_BRICK, cs.PATH_AUTO, cs.PATH_SLAB])
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_packed_format_round_trip(name, path):
    gd = load_golden(name)
    M, K = int(gd["M"]), int(gd["K"])
    p = cs.Plan(M, K, gd["row_ptr"], gd["cols"], gd["vals"], host_only=True, path=path, split_nnz=16)
    rp, cols, vals = p.decode_csr()
    # expected: the input with every row sorted by column
    exp_c, exp_v = gd["cols"].copy(), gd["vals"].copy()
    for r in range(M):
        j0, j1 = int(gd["row_ptr"][r]), int(gd["row_ptr"][r + 1])
        o = np.argsort(exp_c[j0:j1], kind="stable")
        exp_c[j0:j1], exp_v[j0:j1] = exp_c[j0:j1][o], exp_v[j0:j1][o]
    assert np.array_equal(rp, gd["row_ptr"].astype(np.uint64))
    assert np.array_equal(cols, exp_c)
    assert np.array_equal(vals.view(np.uint32), exp_v.view(np.uint32))


def test_round_trip_partial_last_panel_and_empty():
    A = g.uniform_random(37, 50, 3, seed=3)  # M not a multiple of 16
    for path in (cs.PATH_ROWS, cs.PATH_BRICK, cs.PATH_SLAB):
        p = cs.Plan.from_csr(A, host_only=True, path=path)
        rp, cols, vals = p.decode_csr()
        assert np.array_equal(cols, A.cols.numpy().astype(np.uint32))
        assert p.info()["num_panels"] == 3
    empty = cs.Plan(32, 32, np.zeros(33, np.uint64), np.zeros(0, np.uint32), np.zeros(0, np.float32), host_only=True)
    assert empty.info()["nnz"] == 0 and empty.info()["num_blocks"] == 0
    zero_rows = cs.Plan(0, 8, np.zeros(1, np.uint64), np.zeros(0, np.uint32), np.zeros(0, np.float32), host_only=True)
    assert zero_rows.info()["num_panels"] == 0


def test_long_rows_become_chunks():
    gd = load_golden("rmat_s8")
    p = cs.Plan(int(gd["M"]), int(gd["K"]), gd["row_ptr"], gd["cols"], gd["vals"], host_only=True, path=cs.PATH_ROWS,
                split_nnz=8)
    lens = np.diff(gd["row_ptr"].astype(np.int64))
    info = p.info()
    assert info["num_long_rows"] == int((lens > 8).sum())
    assert info["num_chunks"] == int(np.ceil(lens[lens > 8] / 8).sum())


def _plan_of_row_lengths(lens, **kw):
    lens = np.asarray(lens, np.int64)
    rp = np.zeros(lens.size + 1, np.uint64)
    np.cumsum(lens, out=rp[1:])
    cols = np.concatenate([np.arange(l, dtype=np.uint32) for l in lens]) if lens.sum() else np.zeros(0, np.uint32)
    return cs.Plan(lens.size, int(max(lens.max(), 1)), rp, cols, np.ones(cols.size, np.float32), host_only=True, path=cs.PATH_ROWS, **kw)


def test_sizes_left_to_the_library_follow_the_job():
    """split_nnz = tile_nnz = 0: a small job gets tiles for one resident wave, rows are cut from 128 nonzeros on and
    a cut row into pieces of ceil(sqrt(length / 2)) (at least 32) nonzeros; a large job keeps 256 / 512; given values
    are taken as given."""
    chunks = lambda lens, **kw: (lambda i: (i["num_long_rows"], i["num_chunks"]))(_plan_of_row_lengths(lens, **kw).info())
    assert chunks([128]) == (0, 0)                       # not longer than the cut length
    assert chunks([130]) == (1, 5)                       # pieces of 32
    assert chunks([2400]) == (1, 69)                     # pieces of ceil(sqrt(1200)) = 35
    assert chunks([2400], split_nnz=256) == (1, 10)      # as given
    assert chunks([2400], tile_nnz=512) == (1, 10)       # one of the two given: the other takes its large-job default
    # 4000 rows of 4 nonzeros: cost 32 000 -> tiles of the smallest cost (96 = 12 rows); with the default cost 512, 64 rows each
    small = [4] * 4000
    assert _plan_of_row_lengths(small).info()["num_tiles"] == -(-4000 // 12)
    assert _plan_of_row_lengths(small, tile_nnz=512, split_nnz=256).info()["num_tiles"] == -(-4000 // 64)
    # a large job (cost above 2.1 M): 256-nonzero chunks, tiles of cost 512
    big = [8] * 200_000 + [3000]
    info = _plan_of_row_lengths(big).info()
    assert (info["num_long_rows"], info["num_chunks"]) == (1, 12)
    assert info["num_tiles"] == -(-200_000 // 43)        # 43 rows x (8 + 4) reach cost 512


def test_bad_input_is_rejected_not_fatal():
    rp = np.array([0, 2, 1], np.uint64)
    with pytest.raises(cs.CuteSpmmError) as e:
        cs.Plan(2, 4, rp, np.zeros(2, np.uint32), np.zeros(2, np.float32), host_only=True)
    assert e.value.status == -1
    with pytest.raises(cs.CuteSpmmError) as e:  # column index >= K
        cs.Plan(1, 4, np.array([0, 1], np.uint64), np.array([4], np.uint32), np.ones(1, np.float32), host_only=True)
    assert e.value.status == -1 and "column" in str(e.value)
    with pytest.raises(cs.CuteSpmmError):  # rowPtr[0] != 0
        cs.Plan(1, 4, np.array([1, 1], np.uint64), np.zeros(1, np.uint32), np.ones(1, np.float32), host_only=True)
    h = ctypes.c_void_p()
    assert cs.lib.cutespmm_plan_build_host(ctypes.byref(h), 1, 1, None, None, None, None) == -1
    assert cs.lib.cutespmm_plan_info(None, None) == -1


def test_host_only_plan_refuses_to_execute():
    gd = load_golden("stencil_16x16")
    p = cs.Plan(int(gd["M"]), int(gd["K"]), gd["row_ptr"], gd["cols"], gd["vals"], host_only=True)
    st = cs.lib.cutespmm_spmm(p._h, 16, 16, 16, 16, 16, None)
    assert st == -4  # unsupported: there is no CPU execution path


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_plan_create_without_gpu_fails_loudly():
    gd = load_golden("stencil_16x16")
    with pytest.raises(cs.CuteSpmmError) as e:
        cs.Plan(int(gd["M"]), int(gd["K"]), gd["row_ptr"], gd["cols"], gd["vals"])
    assert e.value.status == -3


@pytest.mark.parametrize("name", ["general_5x7", "symmetric_20"])
def test_mtx_reader_matches_reference(name):
    gd = dict(np.load(GOLDEN / f"mtx_{name}.npz"))
    r = cs.MtxReader(GOLDEN / f"{name}.mtx")
    assert (r.M, r.K, r.nnz) == (int(gd["M"]), int(gd["K"]), int(gd["nnz"]))
    assert np.array_equal(r.rowPtr, gd["row_ptr"])
    assert np.array_equal(r.cols, gd["cols"])
    assert np.array_equal(r.vals, gd["vals"])


def test_mtx_reader_keeps_values_when_asked_and_reports_missing_file():
    r = cs.MtxReader(GOLDEN / "general_5x7.mtx", pattern_only=False)
    assert sorted(r.vals.tolist())[0] == -2.0 and 9.0 in r.vals
    with pytest.raises(cs.CuteSpmmError) as e:
        cs.MtxReader(GOLDEN / "does_not_exist.mtx")
    assert e.value.status == -5


def test_mtx_reader_rejects_malformed_files_with_a_message(tmp_path):
    """Malformed files end in CUTESPMM_EIO with the path and line in the last-error string, never in an
    out-of-range write: a mirrored entry outside a non-square "symmetric" matrix, and an entry line with one
    number (which must not borrow the next line's first number)."""
    f = tmp_path / "sym_nonsquare.mtx"
    f.write_text("%%MatrixMarket matrix coordinate real symmetric\n3 40 2\n1 1 1.0\n2 35 1.0\n")
    with pytest.raises(cs.CuteSpmmError) as e:
        cs.MtxReader(f)
    assert e.value.status == -5
    msg = cs.lib.cutespmm_last_error().decode()
    assert "sym_nonsquare.mtx" in msg and "line 4" in msg
    f2 = tmp_path / "one_number.mtx"
    f2.write_text("%%MatrixMarket matrix coordinate pattern general\n4 4 2\n3\n2 2\n")
    with pytest.raises(cs.CuteSpmmError):
        cs.MtxReader(f2)
    assert "line 3" in cs.lib.cutespmm_last_error().decode()
    with pytest.raises(cs.CuteSpmmError):
        cs.MtxReader(tmp_path / "missing.mtx")
    assert "cannot open" in cs.lib.cutespmm_last_error().decode()


def test_partition_rows_balances_nnz_and_aligns():
    A = g.rmat(12, 8, seed=5)
    rp = A.row_ptr.numpy().astype(np.uint64)
    for parts in (1, 2, 3, 8):
        b = cs.partition_rows(rp, parts, align_rows=16)
        assert b[0] == 0 and b[-1] == A.M and np.all(np.diff(b.astype(np.int64)) >= 0)
        assert np.all(b[1:-1] % 16 == 0)
        cost = (rp[b[1:].astype(np.int64)] - rp[b[:-1].astype(np.int64)]).astype(np.float64) + 4.0 * np.diff(b.astype(np.int64))
        assert cost.max() <= 1.25 * cost.mean() + 16 * 40
    # more parts than panels: empty ranges allowed, still monotone
    b = cs.partition_rows(np.array([0, 1, 2], np.uint64), 4, align_rows=16)
    assert b[0] == 0 and b[-1] == 2 and np.all(np.diff(b.astype(np.int64)) >= 0)



def _shuffle_rows(A, seed=5):
    """P*A: the same rows in a random order (columns untouched)."""
    perm = torch.randperm(A.M, generator=torch.Generator().manual_seed(seed))
    lens = (A.row_ptr[1:] - A.row_ptr[:-1])[perm]
    rp = torch.zeros(A.M + 1, dtype=torch.int64)
    torch.cumsum(lens, 0, out=rp[1:])
    idx = torch.repeat_interleave(A.row_ptr[:-1][perm] - rp[:-1], lens) + torch.arange(int(rp[-1]))
    return g.CsrMatrix(A.M, A.K, rp, A.cols[idx], A.vals[idx], A.name + "_shuffled"), perm


@pytest.mark.parametrize("how", ["cluster", "similar"])
@pytest.mark.parametrize("path", [cs.PATH_ROWS, cs.PATH_BRICK, cs.PATH_AUTO])
def test_row_clustering_round_trip_and_effect(path, how):
    """CUTESPMM_REORDER_CLUSTER_ROWS changes the order rows are processed in, nothing else: the plan decodes to the
    caller's matrix in the caller's row order.  On a stencil whose rows were shuffled it brings similar rows back
    together, so the panels are dense enough for the tensor-core kernel again."""
    S, _ = _shuffle_rows(g.stencil9(48))
    for A in (S, g.rmat(10, 8, seed=3, values="uniform"), g.uniform_random(100, 64, 3, seed=8)):
        p = cs.Plan.from_csr(A, path=path, reorder=how, host_only=True)
        rp, cols, vals = p.decode_csr()
        assert np.array_equal(rp, A.row_ptr.numpy().astype(np.uint64))
        assert np.array_equal(cols, A.cols.numpy().astype(np.uint32)) and np.array_equal(vals, A.vals.numpy())
    if path == cs.PATH_AUTO:
        plain = cs.Plan.from_csr(S, host_only=True).info()
        clustered = cs.Plan.from_csr(S, reorder=how, host_only=True).info()
        ordered = cs.Plan.from_csr(g.stencil9(48), host_only=True).info()
        assert plain["brick_panels"] == 0                    # 16 random rows share no columns: no panel is dense enough
        assert clustered["brick_panels"] >= 0.9 * ordered["brick_panels"] > 0
        assert clustered["num_blocks"] < 0.5 * plain["num_blocks"]  # far fewer active-column blocks per panel


def test_row_clustering_is_refused_where_it_is_not_built():
    A = g.stencil9(16)
    with pytest.raises(cs.CuteSpmmError) as e:
        cs.Plan.from_csr(A, path=cs.PATH_SLAB, reorder="cluster", host_only=True)
    assert e.value.status == -4
    with pytest.raises(cs.CuteSpmmError) as e:
        cs.Plan.from_csr(A, reorder=7, host_only=True)
    assert e.value.status == -1


@pytest.mark.parametrize("kw", [dict(path=cs.PATH_AUTO), dict(path=cs.PATH_ROWS, split_nnz=32), dict(path=cs.PATH_SLAB),
                                dict(path=cs.PATH_AUTO, reorder="cluster")])
def test_plan_save_and_load_round_trip(tmp_path, kw):
    """A saved plan loads back to the same description and the same matrix; a damaged, cut or foreign file is refused."""
    A = g.stencil9(40) if kw.get("path") != cs.PATH_ROWS else g.rmat(10, 8, seed=2, values="uniform")
    p = cs.Plan.from_csr(A, host_only=True, **kw)
    f = tmp_path / "plan.bin"
    p.save(f)
    q = cs.Plan.load(f, host_only=True)
    assert q.info() == p.info() and (q.M, q.K, q.nnz) == (A.M, A.K, A.nnz)
    for a, b in zip(p.decode_csr(), q.decode_csr()):
        assert np.array_equal(a, b)
    assert np.array_equal(p.blocked_row_ptr(), q.blocked_row_ptr()) and np.array_equal(p.active_cols(), q.active_cols())
    raw = bytearray(f.read_bytes())
    raw[len(raw) // 2] ^= 0x40
    (tmp_path / "flipped.bin").write_bytes(raw)
    (tmp_path / "cut.bin").write_bytes(bytes(raw[: len(raw) // 3]))
    (tmp_path / "foreign.bin").write_bytes(b"%%MatrixMarket matrix coordinate real general\n")
    for name in ("flipped.bin", "cut.bin", "foreign.bin", "missing.bin"):
        with pytest.raises(cs.CuteSpmmError) as e:
            cs.Plan.load(tmp_path / name, host_only=True)
        assert e.value.status == -5, name


def test_similar_rows_grouping_shrinks_the_panels_column_sets():
    """CUTESPMM_REORDER_SIMILAR_ROWS grows each 16-row panel as a compact patch of the matrix graph: on a 2-D stencil in
    natural order (16 consecutive grid points per panel: 3 x 18 columns) and on the block-structured 3-D matrix the
    panels name clearly fewer distinct columns, i.e. fewer tensor-core bricks and fewer gathered rows of B."""
    for A, gain in ((g.stencil9(96), 0.80), (g.elasticity3d(12, 3, 2), 0.90)):
        plain = cs.Plan.from_csr(A, host_only=True).info()
        grouped = cs.Plan.from_csr(A, reorder="similar", host_only=True).info()
        assert grouped["num_bricks"] <= gain * plain["num_bricks"], (A.name, plain["num_bricks"], grouped["num_bricks"])
        assert grouped["nnz"] == plain["nnz"]


def test_kernels_of_a_product_by_width():
    """Path auto runs the brick kernel from 64 columns on and the row kernel alone below; path brick runs bricks at every
    width the brick kernel takes (multiples of 32); widths it does not take fall to the row kernel's all-rows list."""
    gd = load_golden("stencil_16x16")
    mk = lambda **kw: cs.Plan(int(gd["M"]), int(gd["K"]), gd["row_ptr"], gd["cols"], gd["vals"], host_only=True, **kw)
    auto, brick, rows = mk(path=cs.PATH_AUTO, min_brick_panels=1), mk(path=cs.PATH_BRICK), mk(path=cs.PATH_ROWS)
    assert auto.info()["num_bricks"] > 0
    assert [auto.kernels(n) for n in (16, 32, 48, 64, 128, 100, 512, 576)] == ["rows", "rows", "rows", "brick", "brick", "rows", "brick", "brick"]
    assert [brick.kernels(n) for n in (32, 64, 48)] == ["brick", "brick", "rows"]
    assert [rows.kernels(n) for n in (32, 128)] == ["rows", "rows"]
    assert auto.launch_count(32) == 1 and auto.launch_count(128) == 1 and auto.launch_count(1024) == 2


def test_auto_keeps_small_matrices_on_the_row_kernel():
    """The default of path auto: dense panels go to the tensor-core kernel only when there are enough of them to fill
    its grid (4440); a small stencil stays on the row kernel, the 512 x 512 one does not."""
    small, big = g.stencil9(96), g.stencil9(512)
    assert cs.Plan.from_csr(small, host_only=True, min_brick_panels=4440).info()["brick_panels"] == 0
    assert cs.Plan.from_csr(small, host_only=True, min_brick_panels=1).info()["brick_panels"] == small.M // 16
    cs.default_min_brick_panels = 0  # the library's own default
    assert cs.Plan.from_csr(small, host_only=True).info()["brick_panels"] == 0
    assert cs.Plan.from_csr(big, host_only=True).info()["brick_panels"] == big.M // 16
    assert cs.Plan.from_csr(small, host_only=True, path=cs.PATH_BRICK).info()["brick_panels"] == small.M // 16  # an explicit path is obeyed
