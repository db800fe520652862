"""Extracts the parameter lists of the reference's own tests into tests/golden/reference_case_lists.json.

    python tests/golden/make_case_lists.py /path/to/flash-attention-npu

The reference's test modules cannot be imported without its device package, and they re-bind one module-level name
(`test_cases`) for several lists, so the lists are read from the source with `ast`: every list literal assigned at
module level is attached to the next `test_*` function that follows it, together with the argument names of that
function's `parametrize` decorators.  Only the parameter tuples are taken (shapes, flags, dtypes as text); the test
logic here is this repository's own (tests/test_reference_case_lists_gpu.py)."""
import ast
import json
import os
import sys

FILES = ["test_flash_attn_npu_v2.py", "test_flash_attn_npu_v2_bwd.py", "test_flash_attn_npu_v3.py",
         "test_flash_attn_npu_v3_bwd.py"]


def literal(node):
    """Python value of a tuple / constant node; `torch.bfloat16` becomes the text "bfloat16"."""
    if isinstance(node, ast.Tuple) or isinstance(node, ast.List):
        return [literal(e) for e in node.elts]
    if isinstance(node, ast.Attribute):
        return node.attr
    if isinstance(node, ast.UnaryOp) and isinstance(node.op, ast.USub):
        return -literal(node.operand)
    return ast.literal_eval(node)


def extract(path):
    with open(path) as f:
        tree = ast.parse(f.read())
    lists, pending = {}, {}
    for node in tree.body:
        if isinstance(node, ast.Assign) and isinstance(node.value, ast.List) and node.value.elts and \
                isinstance(node.value.elts[0], ast.Tuple):
            for t in node.targets:
                if isinstance(t, ast.Name):
                    pending[t.id] = (node.lineno, literal(node.value))
        if isinstance(node, ast.FunctionDef) and node.name.startswith("test"):
            for dec in node.decorator_list:
                if not (isinstance(dec, ast.Call) and ast.unparse(dec.func).endswith("parametrize")):
                    continue
                names, values = dec.args[0], dec.args[1]
                if isinstance(values, ast.Name) and values.id in pending:
                    line, cases = pending[values.id]
                    lists[node.name] = {"source": f"tests/{os.path.basename(path)}:{line}",
                                        "fields": [s.strip() for s in ast.literal_eval(names).split(",")],
                                        "cases": cases}
                elif isinstance(values, ast.List):
                    lists.setdefault(node.name + "/extra", {})[ast.literal_eval(names)] = literal(values)
    return lists


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_case_lists.py <checkout of the reference project>")
    ref = sys.argv[1]
    out = {}
    for name in FILES:
        out[name[:-3]] = extract(os.path.join(ref, "tests", name))
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_case_lists.json")
    with open(dst, "w") as f:
        json.dump(out, f, separators=(",", ":"))
    for mod, lists in out.items():
        for fn, d in lists.items():
            print(mod, fn, len(d["cases"]) if "cases" in d else d)


if __name__ == "__main__":
    main()
