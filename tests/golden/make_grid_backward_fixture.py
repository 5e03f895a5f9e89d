"""Writes grid_backward_handcheck.json: a 2-level, 2-D dense grid small enough to check by hand, with the parameter
gradient of a few samples derived here by explicit enumeration of the four corners of every (sample, level) - plain
Python arithmetic following the published definition of the encoding's backward pass
(include/encodings/grid.h:137-245: pos = scale * x + 0.5, g = floor(pos), w = pos - g,
grad[level][index(g + c)][f] += prod_d (c_d ? w_d : 1 - w_d) * dL/dy[level * F + f]; dense index
g_0 + g_1 * resolution, include/common/common_device.h:737-765; level sizes and scales
include/encodings/grid.h:613-641, common_device.h:767-775).  It does not use the oracle, so it pins the oracle
(and through it the CUDA kernels), which the reference's own tests cannot: their backward fixtures are CSV files
that are not part of the reference repository (test/doctest_encodings.cpp:76-154).

Worked by hand for the first sample x = (0.5, 0.5), dL/dy = (1, 2 | 3, 4):
  level 0: scale = 4 * 2^0 - 1 = 3, resolution = 4, 16 entries.  pos = (2, 2), w = (0, 0): all weight on vertex
           (2, 2) = entry 2 + 2 * 4 = 10            -> grad[10] = (1, 2)
  level 1: scale = 4 * 2^1 - 1 = 7, resolution = 8, 64 entries after the 16 of level 0.  pos = (4, 4), w = (0, 0):
           vertex (4, 4) = entry 16 + 4 + 4 * 8 = 52 -> grad[52] = (3, 4)
and for the second, x = (0.25, 0.75), dL/dy = (1, 0 | 0, 0), level 0: pos = (1.25, 2.75), g = (1, 2), w = (0.25, 0.75):
  entries 9, 10, 13, 14 receive 0.1875, 0.0625, 0.5625, 0.1875.

Run from the repository root:  python tests/golden/make_grid_backward_fixture.py
"""
import json
import math
import os

CONFIG = dict(n_dims_to_encode=2, n_levels=2, n_features_per_level=2, log2_hashmap_size=10, base_resolution=4,
              per_level_scale=2.0, type="Dense", interpolation="Linear")
SAMPLES = [  # (x, dL/dy over the 4 feature columns); binary fractions keep every product exact in fp32
    ((0.5, 0.5), (1.0, 2.0, 3.0, 4.0)),
    ((0.25, 0.75), (1.0, 0.0, 0.0, 0.0)),
    ((0.125, 0.625), (-0.5, 0.25, 2.0, -1.0)),
    ((0.875, 0.0625), (0.75, -2.0, 0.5, 1.5)),
    ((0.25, 0.75), (0.5, 0.5, -1.0, 1.0)),  # same cell as the second sample: contributions add up
]


def levels():
    out, offset = [], 0
    for l in range(CONFIG["n_levels"]):
        scale = 2.0 ** (l * math.log2(CONFIG["per_level_scale"])) * CONFIG["base_resolution"] - 1.0
        res = math.ceil(scale) + 1
        n = (res ** 2 + 7) // 8 * 8
        out.append((scale, res, offset, n))
        offset += n
    return out, offset


def main():
    lv, n_entries = levels()
    F = CONFIG["n_features_per_level"]
    grad = [0.0] * (n_entries * F)
    for x, dy in SAMPLES:
        for l, (scale, res, offset, n) in enumerate(lv):
            pos = [scale * x[d] + 0.5 for d in range(2)]
            g = [math.floor(p) for p in pos]
            w = [p - math.floor(p) for p in pos]
            for c in range(4):
                weight, idx, stride = 1.0, 0, 1
                for d in range(2):
                    bit = (c >> d) & 1
                    weight *= w[d] if bit else 1.0 - w[d]
                    idx += (g[d] + bit) * stride
                    stride *= res
                entry = offset + idx % n
                for f in range(F):
                    grad[entry * F + f] += weight * dy[l * F + f]
    assert grad[10 * 2] == 1.0 + 0.0625 + 0.0625 * 0.5 and grad[52 * 2 + 1] == 4.0  # the hand-worked entries
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "grid_backward_handcheck.json")
    json.dump({"config": CONFIG, "n_params": n_entries * F, "x": [s[0] for s in SAMPLES], "dy": [s[1] for s in SAMPLES],
               "expected_grad": grad}, open(path, "w"))
    print("wrote", path, n_entries * F, "values")


if __name__ == "__main__":
    main()
