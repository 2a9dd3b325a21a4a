"""Seeded inputs for the code predictor's one-row kernels, in the predictor's fixed shapes (hidden 1024, SwiGLU 3072,
16 query / 8 KV heads of 128, at most 16 cached positions; 17.cu:7991-8004).  Shared by the tests and by the script
that produced the golden outputs of the reference's own kernels; the weights are regenerated from the seeds, only
the reference's outputs are stored."""
import numpy as np

from oracle import qm_oracle as oracle

HIDDEN, INTERMEDIATE, HQ, HKV, D, MAX_CACHE = 1024, 3072, 16, 8, 128, 16
QD, KD = HQ * D, HKV * D


class PredictorCase:
    def __init__(self, seed):
        s = seed * 1000
        self.seed = seed
        self.x = oracle.normal_bf16(s + 1, (HIDDEN,))
        self.q_w = oracle.scaled_normal_bf16(s + 2, (QD, HIDDEN), 0.03)
        self.k_w = oracle.scaled_normal_bf16(s + 3, (KD, HIDDEN), 0.03)
        self.v_w = oracle.scaled_normal_bf16(s + 4, (KD, HIDDEN), 0.03)
        self.o_w = oracle.scaled_normal_bf16(s + 5, (HIDDEN, QD), 0.02)
        self.context = oracle.normal_bf16(s + 6, (QD,))
        self.attention = oracle.scaled_normal_bf16(s + 7, (HIDDEN,), 0.5)
        self.post_norm_w = oracle.f32_to_bf16(1.0 + 0.1 * oracle.bf16_to_f32(oracle.normal_bf16(s + 8, (HIDDEN,))))
        self.gate_w = oracle.scaled_normal_bf16(s + 9, (INTERMEDIATE, HIDDEN), 0.03)
        self.up_w = oracle.scaled_normal_bf16(s + 10, (INTERMEDIATE, HIDDEN), 0.03)
        self.down_w = oracle.scaled_normal_bf16(s + 11, (HIDDEN, INTERMEDIATE), 0.02)
        self.act = oracle.normal_bf16(s + 12, (INTERMEDIATE,))
        self.residual = oracle.normal_bf16(s + 13, (HIDDEN,))
        # attention path: pre-norm q / k / v of the new token, head norm weights, a cache filled up to each position
        self.q = oracle.normal_bf16(s + 14, (HQ, D))
        self.k = oracle.normal_bf16(s + 15, (HKV, D))
        self.v = oracle.normal_bf16(s + 16, (HKV, D))
        self.q_norm_w = oracle.f32_to_bf16(1.0 + 0.25 * oracle.bf16_to_f32(oracle.normal_bf16(s + 17, (D,))))
        self.k_norm_w = oracle.f32_to_bf16(1.0 + 0.25 * oracle.bf16_to_f32(oracle.normal_bf16(s + 18, (D,))))
        self.cos, self.sin = oracle.make_rope(MAX_CACHE)
        # what earlier positions left in the caches [8][16][128]: K as the kernels store it (normed, roped), V raw
        k_prev = oracle.normal_bf16(s + 19, (MAX_CACHE, HKV, D))
        v_prev = oracle.normal_bf16(s + 20, (MAX_CACHE, HKV, D))
        self.key_cache = np.zeros((HKV, MAX_CACHE, D), dtype=np.uint16)
        self.value_cache = np.zeros_like(self.key_cache)
        oracle.append(np.zeros((MAX_CACHE, HQ, D), dtype=np.uint16), k_prev, v_prev, self.q_norm_w, self.k_norm_w, self.cos,
                      self.sin, 0, self.key_cache, self.value_cache)

    def caches_before(self, position):
        """The caches as they are when the token at `position` arrives: positions >= position still empty."""
        kc, vc = self.key_cache.copy(), self.value_cache.copy()
        kc[:, position:] = 0
        vc[:, position:] = 0
        return kc, vc


SEEDS = (401, 402)
POSITIONS = (0, 1, 6, 15)          # cache_position of the new token; it then attends position + 1 keys
