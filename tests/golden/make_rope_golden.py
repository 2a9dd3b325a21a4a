"""Writes tests/golden/rope_rows_golden.npz from the reference's own host function make_talker_rope
(devices/rtx4090-24g/qwen3_tts_1_7b.cu:21758-21772), called through oracle/_ref/libqm_refkernels.so.
Needs no GPU.  Run from the repository root:  python tests/golden/make_rope_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import qm_oracle as oracle  # noqa: E402

rows, start = 96, 4000
cos, sin = oracle.ref_make_rope(rows, start)
np.savez_compressed(Path(__file__).with_name("rope_rows_golden.npz"), rows=rows, start=start, cos=cos, sin=sin)
print("written", cos.shape)
