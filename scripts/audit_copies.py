"""Static audit for hidden tensor copies in the hot Python files.

    python scripts/audit_copies.py [files...]

Walks the AST and reports calls that materialise a new tensor where a view or a fused kernel could
do: ``.contiguous() .clone() .to() .float() .half() .bfloat16() .repeat() .expand_as().contiguous()``,
``torch.cat / stack / pad``, ``permute/transpose`` immediately followed by ``contiguous``, and binary
arithmetic on names that look like activations inside ``forward``-like functions. It cannot know
shapes, so it prints candidates with file:line for a human to judge. Reference counterpart:
scripts/audit_copies.py.
"""

from __future__ import annotations

import ast
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
DEFAULT = ["gdnet_b200/models/gdnet.py", "gdnet_b200/models/layer.py", "gdnet_b200/models/memory.py",
           "gdnet_b200/ops/cuda.py", "gdnet_b200/train/step.py", "gdnet_b200/train/engine.py"]
COPY_METHODS = {"contiguous", "clone", "to", "float", "half", "bfloat16", "double", "repeat", "repeat_interleave"}
COPY_FUNCS = {"cat", "stack", "pad", "concat", "hstack", "vstack"}
LAYOUT = {"permute", "transpose", "t"}
HOT = ("forward", "step", "backward", "read", "write", "trunk", "one_cycle", "projected_step", "_update")


class Audit(ast.NodeVisitor):
    def __init__(self, path: Path):
        self.path, self.stack, self.hits = path, [], []

    def note(self, node, kind, text):
        fn = self.stack[-1] if self.stack else "<module>"
        hot = any(h in fn for h in HOT)
        self.hits.append((node.lineno, kind, fn, hot, text))

    def visit_FunctionDef(self, node):
        self.stack.append(node.name)
        self.generic_visit(node)
        self.stack.pop()

    def visit_Call(self, node):
        f = node.func
        if isinstance(f, ast.Attribute):
            if f.attr in COPY_METHODS:
                inner = f.value
                if f.attr == "contiguous" and isinstance(inner, ast.Call) and isinstance(inner.func, ast.Attribute) \
                        and inner.func.attr in LAYOUT:
                    self.note(node, "layout+copy", f".{inner.func.attr}(...).contiguous()")
                else:
                    self.note(node, "copy", f".{f.attr}()")
            elif f.attr in COPY_FUNCS and isinstance(f.value, ast.Name) and f.value.id in ("torch", "F"):
                self.note(node, "concat", f"{f.value.id}.{f.attr}()")
        self.generic_visit(node)

    def visit_BinOp(self, node):
        if self.stack and any(h in self.stack[-1] for h in HOT) and isinstance(node.op, (ast.Add, ast.Sub, ast.Mult)):
            names = [n.id for n in ast.walk(node) if isinstance(n, ast.Name)]
            if any(n in ("fwd", "side", "x", "c", "logits", "retrieved") for n in names):
                self.note(node, "out-of-place", ast.unparse(node)[:60])


def main() -> int:
    files = [Path(a) for a in sys.argv[1:]] or [ROOT / f for f in DEFAULT]
    total = 0
    for path in files:
        audit = Audit(path)
        audit.visit(ast.parse(path.read_text()))
        hot = [h for h in audit.hits if h[3]]
        print(f"{path.relative_to(ROOT) if path.is_absolute() else path}: {len(audit.hits)} candidates, {len(hot)} in hot functions")
        for line, kind, fn, is_hot, text in sorted(audit.hits):
            print(f"  {'*' if is_hot else ' '} {line:>4} {kind:<12} {fn:<22} {text}")
        total += len(hot)
    print(f"{total} candidates inside hot functions (marked *)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
