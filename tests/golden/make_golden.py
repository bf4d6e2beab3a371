"""Extracts the literal known-answer vectors of dfdx's own tests for the matmul / conv2d path into
JSON fixtures (tests/golden/*.json).  Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/dfdx

The Rust test files are only read as text: for every `#[test] fn`, the nested-array literals passed
to `dev.tensor(...)` and to `assert_close_to_literal!(expr, literal[, tol])` are collected in source
order.  tests/test_golden.py re-states what each test does with those tensors.

Sources (dfdx v0.13.0):
    dfdx-core/src/tensor_ops/matmul/mod.rs      (tests at :327-768)
    dfdx-core/src/tensor_ops/conv2d/tests.rs
    dfdx/src/nn/layers/linear.rs                (tests at :97-204)
    dfdx-core/src/tensor_ops/normalize.rs       (tests at :52-127; the normalisation inside LayerNorm1D)
    dfdx-core/src/tensor_ops/conv1d/tests.rs
    dfdx-core/src/tensor_ops/convtrans2d/tests.rs
    dfdx-core/src/tensor_ops/softmax.rs         (tests at :90-222)
"""
from __future__ import annotations

import ast
import json
import re
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent

FILES = {
    "matmul": "dfdx-core/src/tensor_ops/matmul/mod.rs",
    "conv2d": "dfdx-core/src/tensor_ops/conv2d/tests.rs",
    "linear": "dfdx/src/nn/layers/linear.rs",
    "normalize": "dfdx-core/src/tensor_ops/normalize.rs",
    "conv1d": "dfdx-core/src/tensor_ops/conv1d/tests.rs",
    "convtrans2d": "dfdx-core/src/tensor_ops/convtrans2d/tests.rs",
    "softmax": "dfdx-core/src/tensor_ops/softmax.rs",
}


def _balanced(text: str, start: int, open_ch: str, close_ch: str) -> int:
    """Index just past the bracket that closes text[start] (which must be open_ch)."""
    depth = 0
    for i in range(start, len(text)):
        if text[i] == open_ch:
            depth += 1
        elif text[i] == close_ch:
            depth -= 1
            if depth == 0:
                return i + 1
    raise ValueError("unbalanced")


def _strip_comments(src: str) -> str:
    return re.sub(r"//[^\n]*", "", src)


def _literal(text: str):
    """Parses a Rust nested array literal of floats; None if it is not a pure literal."""
    t = text.strip().lstrip("&").strip()
    if not t.startswith("["):
        return None
    end = _balanced(t, 0, "[", "]")
    body = t[:end]
    if re.search(r"[A-Za-z_]", re.sub(r"[eE][+-]?\d", "", body)):
        return None
    try:
        return ast.literal_eval(body)
    except (ValueError, SyntaxError):
        return None


def _split_args(argtext: str):
    """Splits macro / call arguments at top-level commas."""
    out, depth, cur = [], 0, []
    for ch in argtext:
        if ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
        if ch == "," and depth == 0:
            out.append("".join(cur).strip())
            cur = []
        else:
            cur.append(ch)
    if "".join(cur).strip():
        out.append("".join(cur).strip())
    return out


def extract(src: str) -> dict:
    src = _strip_comments(src)
    consts = {}
    for m in re.finditer(r"const\s+([A-Z_]+)\s*:\s*[^=]+=\s*\[", src):
        start = m.end() - 1
        end = _balanced(src, start, "[", "]")
        consts[m.group(1)] = ast.literal_eval(src[start:end])
    tests = {}
    for m in re.finditer(r"#\[test\]", src):
        fn = re.compile(r"fn\s+(\w+)\s*\(\s*\)\s*\{").search(src, m.end())
        if not fn:
            continue
        body_start = fn.end() - 1
        body = src[body_start:_balanced(src, body_start, "{", "}")]
        events = []
        for ev in re.finditer(r"(dev(?:ice)?\s*\.\s*tensor\s*\(|assert_close_to_literal!\s*\()", body):
            open_idx = ev.end() - 1
            close_idx = _balanced(body, open_idx, "(", ")")
            args = _split_args(body[open_idx + 1:close_idx - 1])
            if ev.group(1).startswith("dev"):
                arg = args[0] if args else ""
                val = consts.get(arg.strip()) if arg.strip() in consts else _literal(arg)
                if val is not None:
                    events.append({"kind": "tensor", "pos": ev.start(), "value": val})
            else:
                if len(args) < 2:
                    continue
                val = _literal(args[1])
                tol = None
                if len(args) > 2:
                    try:
                        tol = float(args[2])
                    except ValueError:
                        tol = None
                events.append({"kind": "assert", "pos": ev.start(), "expr": re.sub(r"\s+", "", args[0]),
                               "value": val, "tol": tol})
        events.sort(key=lambda e: e["pos"])
        for e in events:
            del e["pos"]
        if events:
            tests[fn.group(1)] = events
    return tests


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/dfdx")
    root = Path(sys.argv[1])
    for name, rel in FILES.items():
        tests = extract((root / rel).read_text())
        out = {"source": rel, "tests": tests}
        (HERE / f"{name}.json").write_text(json.dumps(out, indent=1) + "\n")
        n_t = sum(1 for t in tests.values() for e in t if e["kind"] == "tensor")
        n_a = sum(1 for t in tests.values() for e in t if e["kind"] == "assert")
        print(f"{name}: {len(tests)} tests, {n_t} tensors, {n_a} asserts -> {name}.json")


if __name__ == "__main__":
    main()
