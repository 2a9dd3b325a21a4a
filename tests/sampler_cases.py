"""Seeded inputs for the final-head (logits -> code) tests, shared by the golden generator, the CPU pin and the
GPU parity test.  Vocabulary 3072 (the reference's codec vocabulary), EOS 2150, reserved ids from 2048 on."""
import numpy as np

from oracle import qm_oracle as oracle

VOCAB = 3072
EOS = 2150
REPETITION, SUPPRESS, RECORD = 1, 2, 4

# name -> (seed, generation_index, flags, top_k, logit scale)
CASES = {
    "greedy_plain": (11, 0, 0, 0, 4.0),
    "greedy_processed_first_step": (12, 0, REPETITION | SUPPRESS | RECORD, 0, 4.0),
    "greedy_processed_late": (13, 37, REPETITION | SUPPRESS | RECORD, 0, 4.0),
    "greedy_ties": (14, 5, SUPPRESS, 0, 0.05),            # coarse bf16 values: many exactly equal scores
    "topk_plain": (15, 3, 0, 50, 4.0),
    "topk_processed": (16, 120, REPETITION | SUPPRESS | RECORD, 50, 4.0),
    "topk_flat": (17, 9, REPETITION | SUPPRESS, 50, 0.05),
    "topk_eos_window": (18, 1, SUPPRESS | RECORD, 50, 4.0),
}


class SamplerCase:
    def __init__(self, name):
        seed, self.generation_index, self.flags, self.top_k, scale = CASES[name]
        rng = np.random.default_rng(seed)
        values = (rng.standard_normal(VOCAB) * scale).astype(np.float32)
        if name == "greedy_ties":
            values = np.round(values * 64) / 64          # exact ties, also at the maximum
            values[values.argsort()[-7:]] = values.max()
        if name.endswith("eos_window") or name == "greedy_processed_first_step":
            values[EOS] = values.max() + 3.0             # EOS would win if it were allowed
        values[2048 + (seed % 500)] = values.max() + 1.0  # a reserved id that suppression must hide
        self.logits = oracle.f32_to_bf16(values)
        self.history = np.zeros(8192, dtype=np.int32)
        self.history[: self.generation_index] = rng.integers(0, 2048, size=self.generation_index)
        if self.generation_index > 2:
            top = np.argsort(-values[:2048])[:3]
            self.history[:3] = top                        # penalise the leaders so that the penalty matters
        self.rng_state = int(rng.integers(1, 2**62))
        self.temperature = 0.9
