"""Seeded inputs for the non-attention operators of the talker layer (shared by the tests and the golden script)."""
import numpy as np

from oracle import qm_oracle as oracle


class LayerCase:
    """rows token rows in the 1.7B talker widths (hidden 2048), with reduced output widths to keep fixtures small."""

    def __init__(self, seed, rows, hidden=2048, out_features=384, intermediate=320):
        self.seed, self.rows, self.hidden = seed, rows, hidden
        self.x = oracle.normal_bf16(seed * 1000 + 1, (rows, hidden))
        self.attn = oracle.scaled_normal_bf16(seed * 1000 + 2, (rows, hidden), 0.5)
        self.norm_w = oracle.f32_to_bf16(1.0 + 0.1 * oracle.bf16_to_f32(oracle.normal_bf16(seed * 1000 + 3, (hidden,))))
        self.w = oracle.scaled_normal_bf16(seed * 1000 + 4, (out_features, hidden), 0.02)
        self.bias = oracle.scaled_normal_bf16(seed * 1000 + 5, (out_features,), 0.1)
        self.residual = oracle.normal_bf16(seed * 1000 + 6, (rows, out_features))
        self.gate_w = oracle.scaled_normal_bf16(seed * 1000 + 7, (intermediate, hidden), 0.02)
        self.up_w = oracle.scaled_normal_bf16(seed * 1000 + 8, (intermediate, hidden), 0.02)


CASES = {"layer_a": (301, 3), "layer_b": (302, 33)}
