"""Extracts the known-answer vectors that pin the CPU oracle from the reference's own
test programs and writes them to reference_vectors.json (committed beside this script).

Run in a container that has the reference checkout:
    python tests/golden/extract_reference_vectors.py /path/to/reference

Each `.fut` test file carries `-- ==` blocks with `input { ... } output { ... }` pairs
(format: docs/man/futhark-test.rst:20-120 of the reference).  Only blocks with literal
outputs are taken (`auto output` pins nothing).  Values are parsed from the Futhark
value syntax subset these files use: integer and float literals with optional type
suffixes, `true`/`false`, nested arrays, `empty([0]t)`, and `f32.nan`/`f64.nan`/`f32.inf`.
"""
import json
import os
import re
import sys

FILES = [
    "tests/soacs/scan0.fut",
    "tests/soacs/reduce0.fut",
    "tests/soacs/filter1.fut",
    "tests/soacs/partition1.fut",
    "tests/soacs/partition2.fut",
    "tests/soacs/segreduce-iota.fut",
    "tests/hist/simple.fut",
    "tests/hist/max.fut",
    "tests/hist/f32.fut",
    "tests/hist/large.fut",
    "tests/segredomap/segsum-comm.fut",
    "tests/reg-tiling/mmm.fut",
    "tests/mss.fut",
    "tests/soacs/exscan0.fut",
    "tests/soacs/exscan1.fut",
    "tests/modules/functor1.fut",
    "tests/soacs/filter3.fut",
    "tests/soacs/scan4.fut",
    "tests/hist/and.fut",
    "tests/hist/or.fut",
    "tests/hist/xor.fut",
    "tests/hist/min.fut",
    "tests/hist/segmented.fut",
    "tests/hist/hist2d.fut",
    "tests/hist/max64.fut",
    "tests/hist/f64.fut",
    "tests/soacs/scan1.fut",
    "tests/soacs/scan3.fut",
    "tests/soacs/mapscan.fut",
    "tests/soacs/scan-with-map.fut",
    "tests/soacs/reduce1.fut",
    "tests/soacs/reduce2.fut",
    "tests/hist/i8.fut",
    "tests/hist/i16.fut",
    "tests/hist/f16.fut",
    "tests/tokens.fut",
    "tests/hist/hist3d.fut",
    "tests/hist/segmented_2d.fut",
    "tests/segredomap/segsum-nocomm.fut",
    "tests/hist/array.fut",
    "tests/hist/array_novec.fut",
    "tests/hist/tuple_partial.fut",
    "tests/soacs/reduce4.fut",
    "tests/soacs/reduce5.fut",
    "tests/hist/lor.fut",
    "tests/hist/equiv.fut",
    "tests/hist/segmented_arr.fut",
    "tests/segredomap/ex1-comm.fut",
    "tests/segredomap/ex1-nocomm.fut",
    "tests/hist/and8.fut",
    "tests/hist/and16.fut",
    "tests/hist/and64.fut",
    "tests/hist/or8.fut",
    "tests/hist/or16.fut",
    "tests/hist/xor8.fut",
    "tests/hist/xor16.fut",
    "tests/hist/xor64.fut",
    "tests/hist/min8.fut",
    "tests/hist/min16.fut",
    "tests/hist/max8.fut",
    "tests/hist/max16.fut",
]

TOKEN = re.compile(r"\s*(empty\(\[[^\]]*\](?:\[[^\]]*\])*\w+\)|f(?:16|32|64)\.nan|f32\.inf|-f32\.inf|true|false|"
                   r"-?\d+\.\d*(?:[eE][-+]?\d+)?(?:f16|f32|f64)?|-?\d+(?:[eE][-+]?\d+)?(?:f16|f32|f64)|"
                   r"-?\d+(?:i8|i16|i32|i64|u8|u16|u32|u64)?|\[|\]|,)")


def tokenize(text):
    pos, out = 0, []
    text = text.strip()
    while pos < len(text):
        m = TOKEN.match(text, pos)
        if not m:
            raise ValueError("cannot tokenize at %r" % text[pos:pos + 30])
        out.append(m.group(1))
        pos = m.end()
    return out


def parse_scalar(tok):
    if tok == "true":
        return True
    if tok == "false":
        return False
    if tok in ("f16.nan", "f32.nan", "f64.nan"):
        return "nan"
    if tok == "f32.inf":
        return "inf"
    if tok == "-f32.inf":
        return "-inf"
    if tok.startswith("empty("):
        return []
    m = re.match(r"(-?[\d.eE+-]+?)(i8|i16|i32|i64|u8|u16|u32|u64|f16|f32|f64)?$", tok)
    num = m.group(1)
    if m.group(2) and m.group(2).startswith("f") or "." in num or "e" in num.lower():
        return float(num)
    return int(num)


def parse_values(tokens):
    """A sequence of top-level values (whitespace separated in the source)."""
    vals, i = [], 0

    def parse_at(i):
        if tokens[i] == "[":
            arr, i = [], i + 1
            while tokens[i] != "]":
                v, i = parse_at(i)
                arr.append(v)
                if tokens[i] == ",":
                    i += 1
            return arr, i + 1
        return parse_scalar(tokens[i]), i + 1

    while i < len(tokens):
        v, i = parse_at(i)
        vals.append(v)
    return vals


def blocks(path):
    """Yields (line_number, input_values, output_values) for literal input/output pairs."""
    lines = open(path).read().split("\n")
    comment = []
    for ln, line in enumerate(lines, 1):
        if line.startswith("--"):
            comment.append((ln, line[2:]))
        else:
            break
    text = "\n".join(t for _, t in comment)
    starts = [ln for ln, _ in comment]
    for m in re.finditer(r"input\s*\{([^{}]*)\}\s*output\s*\{([^{}]*)\}", text, re.S):
        line_no = starts[text.count("\n", 0, m.start())]
        try:
            yield line_no, parse_values(tokenize(m.group(1))), parse_values(tokenize(m.group(2)))
        except ValueError:
            continue


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: extract_reference_vectors.py /path/to/reference")
    ref = sys.argv[1]
    out = {}
    for f in FILES:
        cases = []
        for ln, ins, outs in blocks(os.path.join(ref, f)):
            cases.append({"line": ln, "input": ins, "output": outs})
        out[f] = cases
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.json")
    with open(dst, "w") as fh:
        json.dump(out, fh, indent=1, sort_keys=True)
        fh.write("\n")
    print("wrote", dst, {k: len(v) for k, v in out.items()})


if __name__ == "__main__":
    main()
