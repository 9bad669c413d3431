"""The allocation-free entry point, tc_execute_noalloc.

Some users of the library cannot allocate device memory at call time -- their own pool owns the GPU, or
they sit in a loop that must not synchronise the device -- so this entry takes the scratch of K-sliced
plans from a fixed array inside the library.  Checked here through the C ABI against tc_execute on the
same inputs, twice in a row (the array keeps the previous call's contents), plus its refusals.
Collected last on purpose: a failure here cannot hide the other GPU tests behind `-x`.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LIMIT = 8 << 20  # TC_NOALLOC_MAX_WORKSPACE_BYTES


def test_noalloc_matches_execute_on_two_calls_in_a_row(pkg, orc):
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    # small output, long contraction: the planner slices K, so the kernels need scratch
    expr = "C [a,33,b,17] += sum(c,1000,d,9) * A [a,c,d] * B [d,b,c];"
    c0, a, b = orc.make_inputs(expr, 77)
    ref = orc.contract(expr, c0.copy(), a, b, threads=orc.max_threads())
    plan = pkg.Plan(expr)
    with pytest.raises(pkg.TcError) as e:  # not committed yet: committing allocates, this entry must not
        plan.execute_noalloc(torch.zeros(c0.size, dtype=torch.float64, device="cuda"),
                             torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda())
    assert e.value.status == 7
    plan.commit()
    need = plan.workspace_bytes()
    assert 0 < need <= LIMIT and plan.describe()["ksplit"] > 1
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()

    # The new entry runs FIRST after commit(): committing a K-sliced plan has already resolved the static
    # array's address and loaded the combine kernels, so nothing is left for this call to look up or load.
    got1 = torch.from_numpy(c0).cuda()
    plan.execute_noalloc(got1, da, db)
    got2 = torch.from_numpy(c0).cuda()
    plan.execute_noalloc(got2, da, db)             # second call: the array holds the first call's partials
    want = torch.from_numpy(c0).cuda()
    plan.execute(want, da, db)                     # existing entry point, plan-owned scratch
    torch.cuda.synchronize()
    assert plan.status() == 0
    for got in (got1, got2):
        assert orc.rel_error(got.cpu().numpy(), want.cpu().numpy()) <= 1e-12
        assert orc.rel_error(got.cpu().numpy(), ref) <= 1e-12
    assert np.array_equal(got1.cpu().numpy(), got2.cpu().numpy())

    # accumulating twice through the new entry == twice through the old one
    plan.execute(want, da, db)
    plan.execute_noalloc(got1, da, db)
    torch.cuda.synchronize()
    assert orc.rel_error(got1.cpu().numpy(), want.cpu().numpy()) <= 1e-12
    plan.close()


def test_noalloc_without_scratch_and_refusal_beyond_the_limit(pkg, orc):
    import torch
    torch.cuda.set_device(0)
    # a plan that needs no scratch runs through the same entry
    expr = "C [a,40,b,24,c,12] -= sum(d,20) * A [d,c,a] * B [b,d];"
    c0, a, b = orc.make_inputs(expr, 78, np.float32)
    ref = orc.contract(expr, c0.copy(), a, b)
    plan = pkg.Plan(expr, pkg.F32).commit()
    assert plan.workspace_bytes() == 0
    dc = torch.from_numpy(c0).cuda()
    plan.execute_noalloc(dc, torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda())
    torch.cuda.synchronize()
    assert orc.rel_error(dc.cpu().numpy(), ref) <= 1e-5
    plan.close()
    # scratch beyond the array: refused with a clear status, nothing launched
    big = pkg.Plan("C [a,300,b,300] += sum(c,4096) * A [c,a] * B [c,b];", split_k=64).commit()
    assert big.workspace_bytes() > LIMIT
    buf = torch.zeros(4096 * 300, dtype=torch.float64, device="cuda")
    out = torch.zeros(300 * 300, dtype=torch.float64, device="cuda")
    with pytest.raises(pkg.TcError) as e:
        big.execute_noalloc(out, buf, buf)
    assert e.value.status == 8
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0
    big.close()
