"""Regenerates the golden fixtures in this folder from the reference checkout.

Run in the authoring container only (the reference tree is not present where
the GPU tests run): `python tests/golden/make_golden.py /path/to/reference`.

turbo_codebooks.json: the pre-computed Lloyd-Max centroid table that the
reference ships as data (Libraries/MLXLMCommon/TurboQuantKVCache.swift:57-94),
parsed from the Swift source text. It pins both codebook generators (the
oracle's float32 restatement and the library's double-precision one).
"""
import json
import os
import re
import sys


def parse_codebooks(swift_path: str):
    text = open(swift_path).read()
    start = text.index("private static var precomputed")
    end = text.index("private static let centroidLock")
    block = text[start:end]
    block = block[block.index("= [") + 2:]
    table = {}
    # dim: [ bits: [floats], ... ]
    for dim_match in re.finditer(r"(\d+):\s*\[\s*((?:\d+:\s*\[[^\]]*\],?\s*)+)\]", block):
        dim = dim_match.group(1)
        table[dim] = {}
        for bits_match in re.finditer(r"(\d+):\s*\[([^\]]*)\]", dim_match.group(2)):
            vals = [float(v) for v in bits_match.group(2).replace("\n", " ").split(",") if v.strip()]
            table[dim][bits_match.group(1)] = vals
    return table


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path of the mlx-swift-lm checkout>")
    ref = sys.argv[1]
    here = os.path.dirname(os.path.abspath(__file__))
    table = parse_codebooks(os.path.join(ref, "Libraries/MLXLMCommon/TurboQuantKVCache.swift"))
    for dim, per_bits in table.items():
        for bits, vals in per_bits.items():
            assert len(vals) == 1 << int(bits), (dim, bits, len(vals))
    out = {
        "source": "Libraries/MLXLMCommon/TurboQuantKVCache.swift:57-94 (TurboQuantCodebook.precomputed)",
        "centroids": table,
    }
    with open(os.path.join(here, "turbo_codebooks.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote turbo_codebooks.json:", {d: sorted(b) for d, b in table.items()})


if __name__ == "__main__":
    main()
