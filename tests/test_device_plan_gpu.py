"""cutespmm_plan_create_device: a plan built from CSR arrays that live on the GPU must give the host-built plan's
result bit for bit (same work lists, same packed bricks, same kernels), decode to the arrays it was given, show the
same panel views as the reference's preprocessing, and refuse what the device builder does not do."""
import numpy as np
import pytest
import torch

import cutespmm_ae_b200 as cs
from cutespmm_ae_b200 import generators as g

pytestmark = pytest.mark.gpu


def _dev(A):
    return (A.row_ptr.to(torch.int32).cuda().contiguous(), A.cols.to(torch.int32).cuda().contiguous(), A.vals.to(torch.float32).cuda().contiguous())


@pytest.mark.parametrize("make,N", [(lambda: g.rmat(14, 8, seed=31, values="uniform"), 128), (lambda: g.stencil9(96), 64),
                                     (lambda: g.uniform_random(1000, 777, 5, seed=4), 20)])
def test_device_built_plan_equals_host_built_rows_plan(oracle_mod, make, N):
    A = make()
    rp, cols, vals = _dev(A)
    pd = cs.Plan.from_device_csr(A.M, A.K, rp, cols, vals, path=cs.PATH_ROWS)
    ph = cs.Plan.from_csr(A, path=cs.PATH_ROWS)
    id_, ih = pd.info(), ph.info()
    for k in ("M", "K", "nnz", "num_tiles", "num_long_rows", "num_chunks"):
        assert id_[k] == ih[k]
    assert id_["brick_panels"] == 0
    B = g.dense_operand(A.K, N, 17, device="cuda")
    Cd, Ch = pd.spmm(B), ph.spmm(B)
    torch.cuda.synchronize()
    assert torch.equal(Cd, Ch)
    ref = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, B.cpu().numpy(), A.M, A.K)
    assert oracle_mod.rel_fro(ref, Cd.cpu().numpy()) <= 2e-6
    drp, dcols, dvals = pd.decode_csr()
    assert np.array_equal(drp, A.row_ptr.numpy().astype(np.uint64))
    assert np.array_equal(dcols, A.cols.numpy().astype(np.uint32)) and np.array_equal(dvals, A.vals.numpy())
    assert pd.device_status() == 0


def test_device_builder_handles_unsorted_rows_hub_rows_and_empty_matrices(oracle_mod):
    A = g.rmat(12, 16, seed=9, values="uniform")  # hub rows longer than the split length: chunks + fix-up
    perm = torch.arange(A.nnz)
    rp = A.row_ptr.numpy()
    for r in range(0, A.M, 7):  # reverse the nonzeros of every seventh row: rows need not be sorted
        perm[rp[r]:rp[r + 1]] = torch.arange(rp[r + 1] - 1, rp[r] - 1, -1)
    cols, vals = A.cols[perm], A.vals[perm]
    pd = cs.Plan.from_device_csr(A.M, A.K, A.row_ptr.to(torch.int32).cuda(), cols.to(torch.int32).cuda(), vals.cuda())
    assert pd.info()["num_long_rows"] > 0
    B = g.dense_operand(A.K, 32, 5, device="cuda")
    C = pd.spmm(B).cpu().numpy()
    ref = oracle_mod.spmm_csr(A.row_ptr, cols, vals, B.cpu().numpy(), A.M, A.K)
    assert oracle_mod.rel_fro(ref, C) <= 2e-6
    empty = cs.Plan.from_device_csr(64, 32, torch.zeros(65, dtype=torch.int32, device="cuda"), torch.zeros(0, dtype=torch.int32, device="cuda"),
                                    torch.zeros(0, device="cuda"))
    assert torch.count_nonzero(empty.spmm(torch.ones(32, 8, device="cuda"))) == 0


def test_device_builder_refusals():
    A = g.stencil9(16)
    rp, cols, vals = _dev(A)
    with pytest.raises(cs.CuteSpmmError) as e:
        cs.Plan.from_device_csr(A.M, A.K, rp, cols, vals, path=cs.PATH_SLAB)  # the slab format is built on the host only
    assert e.value.status == -4
    bad_cols = cols.clone()
    bad_cols[5] = A.K  # out of range
    with pytest.raises(cs.CuteSpmmError) as e:
        cs.Plan.from_device_csr(A.M, A.K, rp, bad_cols, vals)
    assert e.value.status == -1
    bad_rp = rp.clone()
    bad_rp[3] = bad_rp[4] + 1  # decreasing
    with pytest.raises(cs.CuteSpmmError) as e:
        cs.Plan.from_device_csr(A.M, A.K, bad_rp, cols, vals)
    assert e.value.status == -1
    p = cs.Plan.from_device_csr(A.M, A.K, rp, cols, vals, path=cs.PATH_ROWS)  # no panel analysis: no panel views
    with pytest.raises(cs.CuteSpmmError) as e:
        p.blocked_row_ptr()
    assert e.value.status == -4
    # a panel beyond the device sort: one row of 9000 nonzeros among short ones
    hrp = torch.zeros(65, dtype=torch.int64)
    hrp[20:] = 9000
    hrp[21:] += torch.arange(1, 45) * 3
    hub = g.CsrMatrix(64, 10000, hrp, torch.cat([torch.arange(9000), torch.arange(132) * 7]).to(torch.int32), torch.ones(9132))
    with pytest.raises(cs.CuteSpmmError) as e:
        cs.Plan.from_device_csr(hub.M, hub.K, *_dev(hub), path=cs.PATH_BRICK)
    assert e.value.status == -4
    auto = cs.Plan.from_device_csr(hub.M, hub.K, *_dev(hub))  # auto: such a panel simply stays with the row kernel
    assert auto.info()["num_long_rows"] == 1
    with pytest.raises(cs.CuteSpmmError):  # ... and the panel views are incomplete
        auto.blocked_row_ptr()


@pytest.mark.parametrize("make,Ns,path", [(lambda: g.stencil9(96), [128, 64, 32, 100], cs.PATH_AUTO),
                                           (lambda: g.elasticity3d(12, 3, 5), [128, 256], cs.PATH_AUTO),
                                           (lambda: g.stencil9(512, 512, 1002), [128], cs.PATH_AUTO),
                                           (lambda: g.uniform_random(777, 555, 9, seed=6), [64], cs.PATH_BRICK),
                                           (lambda: g.rmat(13, 8, seed=12, values="uniform"), [128], cs.PATH_AUTO)])
def test_device_built_tensor_core_plan_equals_host_built(oracle_mod, make, Ns, path):
    """Panel analysis and brick packing on the device: same choice of kernel per panel, same brick stream (bit-identical
    product), same panel views as the host builder, which is itself pinned to the reference's HRPB."""
    A = make()
    pd = cs.Plan.from_device_csr(A.M, A.K, *_dev(A), path=path)
    ph = cs.Plan.from_csr(A, path=path)
    id_, ih = pd.info(), ph.info()
    for k in ("M", "K", "nnz", "num_panels", "num_tiles", "num_long_rows", "num_chunks", "brick_panels", "num_bricks"):
        assert id_[k] == ih[k], k
    if path == cs.PATH_BRICK or "stencil" in A.name or "elasticity" in A.name:
        assert id_["num_bricks"] > 0
    for N in Ns:
        B = g.dense_operand(A.K, N, 19, device="cuda")
        Cd, Ch = pd.spmm(B), ph.spmm(B)
        torch.cuda.synchronize()
        assert torch.equal(Cd, Ch), N
    ref = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, B.cpu().numpy(), A.M, A.K)
    assert oracle_mod.rel_fro(ref, Cd.cpu().numpy()) <= 1e-3
    assert pd.device_status() == 0
    if int((A.row_ptr[1:] - A.row_ptr[:-1]).max()) * 16 <= 8192:  # every panel within the device sort: the views exist
        assert id_["num_blocks"] == ih["num_blocks"]
        assert np.array_equal(pd.blocked_row_ptr(), ph.blocked_row_ptr())
        assert np.array_equal(pd.active_cols(), ph.active_cols())


@pytest.mark.parametrize("name", ["stencil_16x16", "elasticity_4", "uniform_256"])
def test_device_built_views_match_the_reference_preprocessing(name):
    """blockedRowPtr / activeCols of a device-built plan against what the reference's HRPB produced (golden vectors)."""
    from conftest import load_golden

    gd = load_golden(name)
    M, K = int(gd["M"]), int(gd["K"])
    p = cs.Plan.from_device_csr(M, K, torch.from_numpy(gd["row_ptr"].astype(np.int32)).cuda(), torch.from_numpy(gd["cols"].astype(np.int32)).cuda(),
                                torch.from_numpy(gd["vals"]).cuda())
    assert np.array_equal(p.blocked_row_ptr(), gd["blocked_row_ptr"])
    assert np.array_equal(p.active_cols(), gd["active_cols"])


@pytest.mark.parametrize("how", ["host_auto", "host_rows_chunks", "host_slab", "host_clustered", "device_auto", "device_rows"])
def test_saved_plan_gives_the_same_product_after_loading(tmp_path, how):
    """cutespmm_plan_save / cutespmm_plan_load: the loaded plan runs the same kernels on the same arrays (bit-identical C),
    whichever builder made the plan."""
    if how == "host_rows_chunks" or how == "device_rows":
        A = g.rmat(13, 8, seed=15, values="uniform")
    else:
        A = g.stencil9(128)
    if how.startswith("device"):
        p = cs.Plan.from_device_csr(A.M, A.K, *_dev(A), path=cs.PATH_AUTO if how == "device_auto" else cs.PATH_ROWS)
    else:
        kw = {"host_auto": {}, "host_rows_chunks": dict(path=cs.PATH_ROWS, split_nnz=64), "host_slab": dict(path=cs.PATH_SLAB),
              "host_clustered": dict(reorder="cluster")}[how]
        p = cs.Plan.from_csr(A, **kw)
    f = tmp_path / "plan.bin"
    p.save(f)
    q = cs.Plan.load(f)
    ip, iq = p.info(), q.info()
    for k in ("M", "K", "nnz", "num_tiles", "num_chunks", "num_long_rows", "brick_panels", "num_bricks"):
        assert ip[k] == iq[k], k
    B = g.dense_operand(A.K, 128, 23, device="cuda")
    C0, C1 = p.spmm(B), q.spmm(B)
    torch.cuda.synchronize()
    assert torch.equal(C0, C1)
    for a, b in zip(p.decode_csr(), q.decode_csr()):
        assert np.array_equal(a, b)
