"""Seeded cases for the prefill loop's projections (more rows than one 128-row tile; widths that end in the middle
of a 256-column tile), shared by the script that runs the reference's kernels on them and by the tests."""
from oracle import qm_oracle as oracle

# name -> (seed, rows, out_features, in_features)
CASES = {
    "rows150_n192_k256": (7101, 150, 192, 256),
    "rows257_n320_k128": (7102, 257, 320, 128),
    "rows64_n2048_k2048": (7103, 64, 2048, 2048),
}


class ProjectionCase:
    def __init__(self, seed, rows, out_features, in_features):
        self.x = oracle.normal_bf16(seed, (rows, in_features))
        self.w = oracle.scaled_normal_bf16(seed + 1, (out_features, in_features), 0.03)
        self.up_w = oracle.scaled_normal_bf16(seed + 2, (out_features, in_features), 0.03)
        self.bias = oracle.scaled_normal_bf16(seed + 3, (out_features,), 0.1)
        self.residual = oracle.normal_bf16(seed + 4, (rows, out_features))
