"""Writes tests/golden/golden.json: small known-answer vectors for the two paths.

The reference (Rust on a pinned nightly plus the cuda-oxide git dependency)
cannot be built or run in this environment, so these vectors are computed here
by two independent restatements of its CPU references that must agree before
anything is written: the C oracle (oracle/fk_oracle.c) and the pure
numpy/Python formulas in this file, each following examples/src/gemm.rs:434-451,
544-552 and examples/src/flash_forward.rs:326-362, 419-440.

Run from the repository root:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import hashlib
import json
import math
import os
import struct
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def to_bf16(value: float) -> int:
    bits = struct.unpack("<I", struct.pack("<f", value))[0]
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFFFFFF) >> 16


def from_bf16(bits: int) -> float:
    return struct.unpack("<f", struct.pack("<I", bits << 16))[0]


def a_value(row, depth):
    return float((row * 5 + depth * 3) % 7) - 3.0


def b_value(column, depth):
    return float((column * 4 + depth * 5) % 21) - 10.0


def gemm_cells(k):
    """The 7 x 21 distinct dot products, fp32 running sums, and their bf16 roundings."""
    exact, rounded = [], []
    for cell in range(7 * 21):
        total = np.float32(0.0)
        for depth in range(k):
            total = np.float32(total + np.float32(a_value(cell // 21, depth) * b_value(cell % 21, depth)))
        exact.append(float(total))
        rounded.append(to_bf16(float(total)))
    return exact, rounded


def permutation(tensor, head, row, column):
    stride = 11 + 2 * ((row + 17 * tensor) % 63)
    return (53 * head + 37 * row + stride * column + 71 * tensor) % 128


def q_value(head, row, dim):
    return 2.0 if dim == 0 else (permutation(0, head, row, dim) - 64.0) / 64.0


def k_value(head, row, dim):
    return row / 8.0 if dim == 0 else (permutation(1, head, row, dim) - 64.0) / 64.0


def v_value(head, row, dim):
    return 1.0 + permutation(2, head, row, dim) / 64.0


def attention_row(head, row, sequence, scale, causal):
    keys = row + 1 if causal else sequence
    q = [from_bf16(to_bf16(q_value(head, row, d))) for d in range(128)]
    scores = []
    for key in range(keys):
        scores.append(scale * math.fsum(q[d] * from_bf16(to_bf16(k_value(head, key, d))) for d in range(128)))
    top = max(scores)
    weights = [math.exp(s - top) for s in scores]
    total = math.fsum(weights)
    out = [math.fsum(w * from_bf16(to_bf16(v_value(head, key, d))) for key, w in enumerate(weights)) / total
           for d in range(128)]
    return out, top + math.log(total)


def main():
    import oracle

    golden = {"bf16": [], "gemm": {}, "flash": {}}

    for value in [0.0, 1.0, -1.0, 1.00390625, 1.01171875, 3.0e38, 1e-40, -2.5, 0.1, 65504.0, 1.0 + 2 ** -8,
                  1.0 + 3 * 2 ** -9]:
        single = float(np.float32(value))
        assert oracle.to_bf16(single) == to_bf16(single)
        golden["bf16"].append({"value": single, "bits": to_bf16(single)})

    for k in (64, 256, 1088):
        exact, rounded = gemm_cells(k)
        for cell in range(7 * 21):
            assert oracle.gemm_expected(cell // 21, cell % 21, k) == rounded[cell], (k, cell)
        golden["gemm"][str(k)] = {"exact": exact, "bf16": rounded}
    for (m, n, k) in [(512, 256, 256), (768, 1280, 1088)]:
        a, b = oracle.gemm_stage("a", m, k), oracle.gemm_stage("b", n, k)
        assert a[3, 5] == to_bf16(a_value(3, 5)) and b[9, 2] == to_bf16(b_value(9, 2))
        c, _ = oracle.gemm_rows(a, b, 0, m)
        assert oracle.gemm_check_c(c, m, n, k)[0] == 0
        golden["gemm"][f"{m}x{n}x{k}"] = {
            "a_sha256": hashlib.sha256(a.tobytes()).hexdigest(),
            "b_sha256": hashlib.sha256(b.tobytes()).hexdigest(),
            "c_sha256": hashlib.sha256(c.tobytes()).hexdigest(),
        }

    sequence, heads, scale = 256, 2, 0.125
    q, k, v = (oracle.flash_stage(name, sequence, heads) for name in "qkv")
    assert q[1, 7, 9] == to_bf16(q_value(1, 7, 9)) and k[1, 200, 0] == to_bf16(k_value(1, 200, 0))
    assert v[0, 3, 127] == to_bf16(v_value(0, 3, 127))
    golden["flash"]["inputs_sha256"] = {name: hashlib.sha256(t.tobytes()).hexdigest()
                                        for name, t in (("q", q), ("k", k), ("v", v))}
    rows = []
    for head, row, causal in [(0, 0, True), (0, 63, True), (1, 64, True), (1, 255, True), (0, 130, False),
                              (1, 255, False)]:
        out, lse = attention_row(head, row, sequence, scale, causal)
        c_out, c_lse = oracle.flash_rows(q[head], k[head], v[head], row, 1, scale, causal)
        assert np.allclose(c_out[0], out, rtol=1e-12, atol=0), (head, row)
        assert abs(c_lse[0] - lse) < 1e-10
        rows.append({"head": head, "row": row, "causal": causal, "out": out, "lse": lse})
    golden["flash"]["rows"] = rows
    golden["flash"]["sequence"], golden["flash"]["heads"], golden["flash"]["scale"] = sequence, heads, scale

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.json")
    with open(path, "w") as handle:
        json.dump(golden, handle)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
