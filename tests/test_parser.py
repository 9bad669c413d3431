"""The C++ expression front end against the grammar of the reference parser
(cogent/src/algs/bases/tc_gen_inputs.py:28-108) as restated by the CPU checker."""
import random

import pytest


def _random_expr(rng, max_out=6, max_sum=3, multi_char=False):
    """A well-formed binary contraction with random index permutations."""
    letters = list("abcdefghijklmnopqrstuvwxyz")
    rng.shuffle(letters)
    n_out, n_sum = rng.randint(1, max_out), rng.randint(1, max_sum)
    names = letters[:n_out + n_sum]
    if multi_char:
        names = [n + rng.choice(["", "1", "2", "x", "7q"]) for n in names]
    out, sm = names[:n_out], names[n_out:]
    left_ext = [i for i in out if rng.random() < 0.5]
    right_ext = [i for i in out if i not in left_ext]
    left, right = left_ext + sm, right_ext + sm
    rng.shuffle(left)
    rng.shuffle(right)
    ext = {i: rng.randint(1, 9) for i in names}
    op = rng.choice(["+=", "-=", "="])
    tn = rng.sample(["t3", "t2", "v2", "C", "A", "B", "out_1", "X9"], 3)
    semi = rng.choice([";", ""])
    expr = "%s [%s] %s sum(%s) * %s [%s] * %s [%s]%s" % (
        tn[0], ",".join("%s,%d" % (i, ext[i]) for i in out), op, ",".join("%s,%d" % (i, ext[i]) for i in sm),
        tn[1], ",".join(left), tn[2], ",".join(right), semi)
    return expr


def test_product_parser_matches_reference_token_positions(pkg, orc):
    rng = random.Random(7)
    for n in range(300):
        expr = _random_expr(rng, multi_char=(n % 3 == 0))
        mine = pkg.parse(expr)
        ref = orc.parse(expr)
        for k in ("out", "left", "right", "op", "out_idx", "out_ext", "sum_idx", "sum_ext", "left_idx", "right_idx"):
            assert mine[k] == ref[k], (expr, k)


ACCEPTED = [
    "t3 [a,312,b,312,c,24] += sum(d,312) * t2 [b,d,a] * v2 [d,c];",
    "t3 [a,312,b,312,c,24] += sum(d,312) * t2 [b,d,a] * v2 [d,c]",      # ';' is merely stripped
    "t3 [a,16,b,16,c,16] -= sum(d,16) * t2 [d,c,a] * v2 [b,d];",        # '-=' accumulates the negated sum
    "t3 [a,16,b,16,c,16] = sum(d,16) * t2 [d,c,a] * v2 [b,d];",         # '=' overwrites
    "t3 [h1,4,p7,5] += sum(h2,3,p9,2) * t2 [h2,p9,h1] * v2 [p7,p9,h2];",  # multi-character index names
    "  C   [i,64,j,48,k,32]   +=   sum(l,40)   *   A   [l,k,i]   *   B   [j,l]  ;  ",  # any run of blanks
    "anyName [a,2] += sum(b,3) * Other_1 [b,a] * x [b];",               # free tensor names, right operand all-contraction
]

REJECTED = [
    "t3[a,16,b,16] += sum(d,16) * t2 [d,a] * v2 [b,d];",      # name glued to its bracket (IndexError in the reference)
    "t3 [a, 16, b, 16] += sum(d,16) * t2 [d,a] * v2 [b,d];",  # blanks after commas (ValueError in the reference)
    "t3 [a,16,b,16] += sum(d,16)*t2 [d,a]*v2 [b,d];",         # no blanks around '*'
    "t3 [a,b] += sum(d) * t2 [d,a] * v2 [b,d];",              # extents missing (the old grammar without sizes)
    "# t3 [a,16,b,16] += sum(d,16) * t2 [d,a] * v2 [b,d];",   # comment line of the input files
    "t3 [a,16,b,16] *= sum(d,16) * t2 [d,a] * v2 [b,d];",     # unknown operator
    "t3 [a,16,b,16] += total(d,16) * t2 [d,a] * v2 [b,d];",   # not sum(...)
    "t3 [a,16,b,0] += sum(d,16) * t2 [d,a] * v2 [b,d];",      # zero extent
    "t3 [a,16,b,-4] += sum(d,16) * t2 [d,a] * v2 [b,d];",     # negative extent
    "t3 [a,16,b,16] += sum(d,16) * t2 [d,a] * v2 [b,e];",     # unknown index e
    "t3 [a,16,b,16] += sum(d,16) * t2 [d,a] * v2 [b];",       # contraction index missing from one operand
    "t3 [a,16,a,16] += sum(d,16) * t2 [d,a] * v2 [a,d];",     # repeated index
    "t3 [a,16,b,16] += sum(a,16) * t2 [a,b] * v2 [a];",       # index both external and contracted
    "t3 [a,16,b,16,c,4] += sum(d,16) * t2 [d,a] * v2 [b,d];", # output index in no operand
    "",
    "t3 [a,16,b,16] += sum(d,16) * t2 [d,a] * v2 [b,d]; trailing",
]


@pytest.mark.parametrize("expr", ACCEPTED)
def test_accepted_forms(pkg, orc, expr):
    mine = pkg.parse(expr)
    assert mine["out_idx"] == orc.parse(expr)["out_idx"]
    plan = pkg.Plan(expr)
    plan.close()


@pytest.mark.parametrize("expr", REJECTED)
def test_rejected_forms_return_parse_error(pkg, expr):
    with pytest.raises(pkg.TcError) as e:
        pkg.parse(expr)
    assert e.value.status == 1  # TC_ERR_PARSE
    with pytest.raises(pkg.TcError) as e:
        pkg.Plan(expr)
    assert e.value.status == 1


def test_batched_index_is_unsupported_not_a_crash(pkg):
    with pytest.raises(pkg.TcError) as e:
        pkg.parse("t3 [a,4,b,4] += sum(d,4) * t2 [d,a,b] * v2 [b,d];")
    assert e.value.status == 3  # TC_ERR_UNSUPPORTED


# ----------------------------------------------- pinned to the reference's own parser ----
def _golden():
    import json
    import os
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "grammar.json")) as f:
        return json.load(f)


def _same_record(mine, ref):
    """The C++ parser's record against the reference's `temp_target` (tc_gen_inputs.py:108)."""
    assert [mine["out"], mine["left"], mine["right"], mine["op"]] == [ref["out"], ref["left"], ref["right"], ref["op"]]
    for k in ("out_idx", "sum_idx", "left_idx", "right_idx"):
        assert mine[k] == ref[k], k
    assert mine["out_ext"] + mine["sum_ext"] == ref["sizes"]
    assert [[i, e] for i, e in zip(mine["out_idx"] + mine["sum_idx"], mine["out_ext"] + mine["sum_ext"])] == ref["size_pairs"]


def test_every_benchmark_line_parses_as_the_reference_parser_does(pkg, orc):
    """tests/golden/grammar.json holds what tc_gen_Outer_Group (cogent/src/algs/bases/tc_gen_inputs.py:15-147)
    returned for the expression line of each of its 48 input files (made by tests/golden/make_grammar_golden.py)."""
    g = _golden()
    assert len(g["tccg"]) == 48
    for tag, item in sorted(g["tccg"].items()):
        _same_record(pkg.parse(item["line"]), item["parsed"])
        _same_record(orc.parse(item["line"]), item["parsed"])   # the checker's restatement is pinned by the same records
        pkg.Plan(item["line"]).close()


def test_accept_and_reject_where_the_reference_parser_does(pkg):
    for item in _golden()["forms"]:
        ref = item["parsed"]
        if "raises" in ref:   # the reference crashes (IndexError / ValueError): a parse-error status here
            with pytest.raises(pkg.TcError) as e:
                pkg.parse(item["line"])
            assert e.value.status == 1, item["line"]
        else:
            _same_record(pkg.parse(item["line"]), ref)


def test_live_reference_parser_where_its_tree_is_present(pkg):
    """Where the reference tree lies beside the repository, regenerate the records from its parser and compare
    them with the committed file and, on random well-formed lines, with the C++ parser directly."""
    import contextlib
    import importlib.util
    import io
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("make_grammar_golden", os.path.join(here, "golden", "make_grammar_golden.py"))
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    cogent = os.path.join(mk.REF_DEFAULT, "cogent")
    if not os.path.isdir(cogent):
        pytest.skip("reference tree not present")
    import sys
    sys.path.insert(0, cogent)
    try:
        import src.algs.bases.tc_gen_inputs as tgi
    finally:
        sys.path.remove(cogent)
    g = _golden()
    for tag, item in g["tccg"].items():
        assert mk.reference_parse(tgi, item["line"]) == item["parsed"], tag
    rng = random.Random(17)
    for n in range(200):
        expr = _random_expr(rng, multi_char=(n % 3 == 0))
        _same_record(pkg.parse(expr), mk.reference_parse(tgi, expr))
