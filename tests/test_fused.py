"""Several contractions accumulated into one output in one pass (tc_plan_create_fused / tc_execute_fused).

The term lists are the reference's CCSD(T) doubles terms: sd_t_d2 and sd_t_d1
(cogent/input_strings/ccsd_t/original-expressions/sd_t_d2.in:4-30, sd_t_d1.in), written in the expression grammar
with one pair of inputs per term, as the reference's drivers hold them (cogent/drivers/ccsd_t/code_main_sd2_1.c:12-14:
host_t2_1..9, host_v2_1..9).  The checker applies the nine loop nests one after another."""
import numpy as np
import pytest

OUT = "t3 [h3,{h3},h2,{h2},h1,{h1},p6,{p6},p5,{p5},p4,{p4}]"
# (operator, left indices, right indices): which of the output's indices each input of the term carries
SD2 = [("-=", "p7,p4,h1,h2", "p7,h3,p6,p5"), ("-=", "p7,p4,h2,h3", "p7,h1,p6,p5"), ("+=", "p7,p4,h1,h3", "p7,h2,p6,p5"),
       ("+=", "p7,p5,h1,h2", "p7,h3,p6,p4"), ("+=", "p7,p5,h2,h3", "p7,h1,p6,p4"), ("-=", "p7,p5,h1,h3", "p7,h2,p6,p4"),
       ("-=", "p7,p6,h1,h2", "p7,h3,p5,p4"), ("-=", "p7,p6,h2,h3", "p7,h1,p5,p4"), ("+=", "p7,p6,h1,h3", "p7,h2,p5,p4")]
SD1 = [("-=", "h7,p4,p5,h1", "h3,h2,p6,h7"), ("+=", "h7,p4,p5,h2", "h3,h1,p6,h7"), ("-=", "h7,p4,p5,h3", "h2,h1,p6,h7"),
       ("-=", "h7,p5,p6,h1", "h3,h2,p4,h7"), ("+=", "h7,p5,p6,h2", "h3,h1,p4,h7"), ("-=", "h7,p5,p6,h3", "h2,h1,p4,h7"),
       ("+=", "h7,p4,p6,h1", "h3,h2,p5,h7"), ("-=", "h7,p4,p6,h2", "h3,h1,p5,h7"), ("+=", "h7,p4,p6,h3", "h2,h1,p5,h7")]


def _lines(terms, ext, sum_name):
    out = OUT.format(**ext)
    return ["%s %s sum(%s,%d) * t2_%d [%s] * v2_%d [%s];" % (out, op, sum_name, ext[sum_name], k + 1, l, k + 1, r)
            for k, (op, l, r) in enumerate(terms)]


def test_fused_plan_shape_without_a_gpu(pkg):
    ext = dict(h3=16, h2=16, h1=16, p6=24, p5=16, p4=20, p7=24)
    d = pkg.FusedPlan(_lines(SD2, ext, "p7")).describe()
    assert d["terms"] == 9 and d["rank"] == 6 and d["box"] == [4] * 6 and d["box_elems"] == 4096
    assert d["rows_cols"] == [[64, 64]] * 9
    assert d["boxes"] == 4 * 4 * 4 * 6 * 4 * 5
    out = 16 * 16 * 16 * 24 * 16 * 20
    assert d["flops"] == 9 * 2.0 * out * 24
    # the output travels once instead of nine times
    assert d["bytes_term_by_term"] - d["bytes"] == 8 * 2.0 * 8 * out
    # terms must share the output; '=' cannot be fused; more than 64 rows per box is refused
    with pytest.raises(pkg.TcError) as e:
        pkg.FusedPlan(["t3 [a,4,b,4] += sum(c,4) * x [c,a] * y [c,b];", "t3 [b,4,a,4] += sum(c,4) * x [c,a] * y [c,b];"])
    assert e.value.status == 2
    with pytest.raises(pkg.TcError) as e:
        pkg.FusedPlan(["t3 [a,4,b,4] = sum(c,4) * x [c,a] * y [c,b];"])
    assert e.value.status == 3
    one = pkg.FusedPlan(["t3 [a,40,b,40] += sum(c,4) * x [c,a] * y [c,b];"]).describe()
    assert one["box"] == [40, 40] and one["rows_cols"] == [[40, 40]]


@pytest.mark.gpu
@pytest.mark.parametrize("name,terms,sum_name,ext", [
    ("sd2", SD2, "p7", dict(h3=16, h2=16, h1=16, p6=16, p5=16, p4=16, p7=16)),
    ("sd1", SD1, "h7", dict(h3=16, h2=16, h1=16, p6=16, p5=16, p4=16, h7=16)),
    ("sd2 mixed", SD2, "p7", dict(h3=20, h2=16, h1=24, p6=16, p5=20, p4=16, p7=24)),
    ("sd1 ragged", SD1, "h7", dict(h3=10, h2=7, h1=9, p6=6, p5=11, p4=5, h7=13)),
])
def test_fused_terms_against_the_loop_nests(pkg, orc, name, terms, sum_name, ext):
    import torch
    torch.cuda.set_device(0)
    lines = _lines(terms, ext, sum_name)
    n_out = orc.sizes(lines[0])[0]
    c0 = orc.uniform(60, 0, n_out)
    ins = []
    ref = c0.copy()
    for k, line in enumerate(lines):
        _, na, nb = orc.sizes(line)
        a, b = orc.uniform(61 + k, 1, na), orc.uniform(61 + k, 2, nb)
        ins.append((a, b))
        orc.contract(line, ref, a, b, threads=orc.max_threads())   # the nine nests, one after another
    plan = pkg.FusedPlan(lines)
    dc = torch.from_numpy(c0).cuda()
    das = [torch.from_numpy(a).cuda() for a, _ in ins]
    dbs = [torch.from_numpy(b).cuda() for _, b in ins]
    plan.execute(dc, das, dbs)
    torch.cuda.synchronize()
    assert orc.rel_error(dc.cpu().numpy(), ref) <= 1e-12, name
    # the same terms one by one through ordinary plans give the same tensor (up to the order of the additions)
    dc2 = torch.from_numpy(c0).cuda()
    for line, da, db in zip(lines, das, dbs):
        q = pkg.Plan(line)
        q.execute(dc2, da, db)
        q.close()
    torch.cuda.synchronize()
    assert orc.rel_error(dc2.cpu().numpy(), ref) <= 1e-12
    assert orc.rel_error(dc.cpu().numpy(), dc2.cpu().numpy()) <= 1e-12
    plan.close()


@pytest.mark.gpu
def test_fused_terms_with_other_shapes(pkg, orc):
    """Two contraction indices (fastest in different inputs), a 4-D and a 2-D output, odd contraction extents."""
    import torch
    torch.cuda.set_device(0)
    cases = [
        ["C [a,12,b,9,c,10,d,7] += sum(e,5,f,6) * X1 [e,a,f,c] * Y1 [f,b,e,d];",
         "C [a,12,b,9,c,10,d,7] -= sum(e,5,f,6) * X2 [b,e,d,f] * Y2 [e,f,c,a];",
         "C [a,12,b,9,c,10,d,7] += sum(e,5,f,6) * X3 [f,e,a,b] * Y3 [c,d,f,e];"],
        ["C [a,70,b,45] += sum(k,33) * X1 [k,a] * Y1 [k,b];", "C [a,70,b,45] -= sum(k,33) * X2 [a,k] * Y2 [b,k];"],
    ]
    for lines in cases:
        n_out = orc.sizes(lines[0])[0]
        c0 = orc.uniform(70, 0, n_out)
        ref = c0.copy()
        ins = []
        for k, line in enumerate(lines):
            _, na, nb = orc.sizes(line)
            a, b = orc.uniform(71 + k, 1, na), orc.uniform(71 + k, 2, nb)
            ins.append((a, b))
            orc.contract(line, ref, a, b)
        plan = pkg.FusedPlan(lines)
        dc = torch.from_numpy(c0).cuda()
        plan.execute(dc, [torch.from_numpy(a).cuda() for a, _ in ins], [torch.from_numpy(b).cuda() for _, b in ins])
        torch.cuda.synchronize()
        assert orc.rel_error(dc.cpu().numpy(), ref) <= 1e-12, lines[0]
        plan.close()
