"""Makes tests/golden/grammar.json: what the REFERENCE's own parser returns for its grammar fixtures.

Imports tc_gen_Outer_Group (cogent/src/algs/bases/tc_gen_inputs.py:15-147) from the reference tree and runs
it, one line at a time, on
  * the expression line of each of the 48 cogent/input_strings/tccg/input_tccg_NN.in files (read with the
    reference's own reader, tc_gen_helper_GettingInputs, cogent/src/generators/tc_gen_etc.py:4-18, so the
    comment-line rule is the reference's too);
  * the accepted and rejected forms of its whitespace-sensitive grammar (what raises there must be rejected
    by the C++ parser, what parses there must give the same record).
The record kept per line is the reference's `temp_target`: names, index lists, operator and the size pairs.

Usage (where the reference tree is present):  python tests/golden/make_grammar_golden.py [--reference DIR]
"""
import contextlib
import io
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DEFAULT = os.environ.get("TC_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))

FORMS = [
    "t3 [a,312,b,312,c,24] += sum(d,312) * t2 [b,d,a] * v2 [d,c];",
    "t3 [a,312,b,312,c,24] += sum(d,312) * t2 [b,d,a] * v2 [d,c]",
    "t3 [a,312,b,312,c,24] -= sum(d,312) * t2 [b,d,a] * v2 [d,c];",
    "t3 [a,312,b,312,c,24] = sum(d,312) * t2 [b,d,a] * v2 [d,c];",
    "t3 [h1,7,p7,5] += sum(h9,3,p2,4) * t2 [p2,h1,h9] * v2 [h9,p7,p2];",
    "C [i,64,j,48,k,32] += sum(l,40) * A [l,k,i] * B [j,l];",
    "t3[a,312,b,312,c,24] += sum(d,312) * t2 [b,d,a] * v2 [d,c];",
    "t3 [a, 312,b,312,c,24] += sum(d,312) * t2 [b,d,a] * v2 [d,c];",
    "t3 [a,312,b,312,c,24] += sum(d,312)*t2 [b,d,a]*v2 [d,c];",
    "t3 [a,312,b,312,c,24] += sum(d,312) * t2 [b,d,a];",
    "",
]


def reference_parse(mod, line):
    """The reference's record for one line, or the name of the exception it raises."""
    buf = io.StringIO()
    try:
        with contextlib.redirect_stdout(buf):
            groups = mod.tc_gen_Outer_Group([line], -1)
    except Exception as e:  # IndexError / ValueError: the reference crashes on these forms
        return {"raises": type(e).__name__}
    t = groups[0][1][0]
    rec = {"out": t[0], "out_idx": t[1], "op": t[2], "sum_idx": t[3], "left": t[4], "left_idx": t[5], "right": t[6],
           "right_idx": t[7], "size_pairs": t[8], "sizes": t[9]}
    if "ERROR" in buf.getvalue():
        rec["prints_error"] = True
    return rec


def main(reference):
    cogent = os.path.join(reference, "cogent")
    sys.path.insert(0, cogent)
    import src.algs.bases.tc_gen_inputs as tgi       # noqa: E402  (the reference's module)
    import src.generators.tc_gen_etc as etc          # noqa: E402
    out = {"tccg": {}, "forms": []}
    d = os.path.join(cogent, "input_strings", "tccg")
    for f in sorted(os.listdir(d)):
        if not (f.startswith("input_tccg_") and f.endswith(".in")):
            continue
        with contextlib.redirect_stdout(io.StringIO()):
            lines = etc.tc_gen_helper_GettingInputs(os.path.join(d, f))
        assert len(lines) == 1, f
        out["tccg"][f[len("input_tccg_"):-3]] = {"line": lines[0], "parsed": reference_parse(tgi, lines[0])}
    for line in FORMS:
        out["forms"].append({"line": line, "parsed": reference_parse(tgi, line)})
    with open(os.path.join(HERE, "grammar.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    return out


if __name__ == "__main__":
    ref = REF_DEFAULT
    if "--reference" in sys.argv:
        ref = sys.argv[sys.argv.index("--reference") + 1]
    r = main(ref)
    print("%d benchmark lines, %d forms" % (len(r["tccg"]), len(r["forms"])))
