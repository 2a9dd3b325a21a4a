"""One decoder layer of the prefill loop (devices/rtx4090-24g/qwen3_tts_1_7b.cu:16700-16880) on the library's entry
points against the same chain built from the oracle's operators: two packed prompts, reduced widths (hidden 256,
SwiGLU 512), real head shape (16 / 8 heads of 128).  The chain is: input RMSNorm, q / k / v projections, QK-norm +
RoPE + scatter into the paged cache, causal attention, o-projection + residual add, post RMSNorm, gate / up
projections + SwiGLU, down-projection + residual add.  Each materialised tensor of the library's chain is compared
with the oracle's under the chain tolerance; the oracle is fed its own intermediate values, so the comparison at the
end covers the whole layer."""
import numpy as np
import pytest

from oracle import qm_oracle as oracle
import scenario

pytestmark = pytest.mark.gpu

HQ, HKV, D = 16, 8, 128
TOL_MAX_ABS = 2e-2
TOL_MEAN_REL = 1e-2


def close(got_bits, want_bits, scale=1.0):
    m = oracle.error_metrics(oracle.bf16_to_f32(got_bits), oracle.bf16_to_f32(want_bits))
    assert m["max_abs"] <= TOL_MAX_ABS * scale and m["mean_rel"] <= TOL_MEAN_REL * scale, m
    return m


@pytest.mark.parametrize("lengths", [[150, 70], [129, 1, 64]])
def test_prefill_layer_matches_oracle_chain(qm, lengths):
    import torch

    hidden, inter = 256, 512
    nq, nk = HQ * D, HKV * D
    sc = scenario.PrefillScenario(seed=90 + len(lengths), lengths=lengths, random_weights=True)
    total = sc.total
    seed = 9000 + total
    x = oracle.normal_bf16(seed, (total, hidden))
    w = {
        "in_norm": oracle.f32_to_bf16(1.0 + 0.1 * oracle.bf16_to_f32(oracle.normal_bf16(seed + 1, (hidden,)))),
        "post_norm": oracle.f32_to_bf16(1.0 + 0.1 * oracle.bf16_to_f32(oracle.normal_bf16(seed + 2, (hidden,)))),
        "q": oracle.scaled_normal_bf16(seed + 3, (nq, hidden), 0.06), "k": oracle.scaled_normal_bf16(seed + 4, (nk, hidden), 0.06),
        "v": oracle.scaled_normal_bf16(seed + 5, (nk, hidden), 0.06), "o": oracle.scaled_normal_bf16(seed + 6, (hidden, nq), 0.02),
        "k_bias": oracle.scaled_normal_bf16(seed + 7, (nk,), 0.1),
        "gate": oracle.scaled_normal_bf16(seed + 8, (inter, hidden), 0.06), "up": oracle.scaled_normal_bf16(seed + 9, (inter, hidden), 0.06),
        "down": oracle.scaled_normal_bf16(seed + 10, (hidden, inter), 0.04),
    }

    # ---- the oracle's chain
    normed = oracle.rmsnorm(x, w["in_norm"])
    sc.q = oracle.linear(normed, w["q"]).reshape(total, HQ, D)
    sc.k = oracle.linear(normed, w["k"], bias=w["k_bias"]).reshape(total, HKV, D)
    sc.v = oracle.linear(normed, w["v"]).reshape(total, HKV, D)
    context, _ = sc.expected_attention(mode="ref")
    attn = oracle.linear(context.reshape(total, nq), w["o"])
    residual, post = oracle.add_postnorm(x, attn, w["post_norm"])
    act = oracle.gate_up_swiglu(post, w["gate"], w["up"])
    want = oracle.linear(act, w["down"], residual=residual)

    # ---- the library's chain
    def dev(bits):
        return scenario._bf16_tensor(torch, bits)

    eng = qm.TalkerAttention(layers=1, num_pages=sc.num_pages, q_heads=HQ, kv_heads=HKV, max_positions=sc.max_pos)
    try:
        dw = {name: dev(bits) for name, bits in w.items()}
        cu = torch.from_numpy(sc.cu_seqlens).cuda()
        page_table = torch.from_numpy(np.maximum(sc.page_table, 0)).cuda()
        xd = dev(x)
        g_normed = eng.launch_rmsnorm(xd, dw["in_norm"])
        g_q = eng.linear_generic(g_normed, dw["q"])
        g_k = eng.linear_generic(g_normed, dw["k"], bias=dw["k_bias"])
        g_v = eng.linear_generic(g_normed, dw["v"])
        q_rot = eng.prefill_norm_rope_scatter(0, g_q.view(total, HQ, D), g_k.view(total, HKV, D), g_v.view(total, HKV, D),
                                              dev(sc.q_w), dev(sc.k_w), cu, page_table)
        g_context = eng.launch_attention_prefill(0, q_rot, cu, page_table, sc.max_seqlen)
        g_residual = eng.linear_generic(g_context.view(total, nq), dw["o"], residual=xd)
        g_post = eng.launch_rmsnorm(g_residual, dw["post_norm"])
        g_act = eng.gate_up_swiglu_rows(g_post, dw["gate"], dw["up"])
        g_out = eng.linear_generic(g_act, dw["down"], residual=g_residual)
        torch.cuda.synchronize()
        assert eng.status() == 0
        bits = scenario._bits
        close(bits(g_q), sc.q.reshape(total, nq), scale=2.0)
        close(bits(g_k), sc.k.reshape(total, nk), scale=2.0)
        close(bits(g_context), context, scale=2.0)
        close(bits(g_residual), residual, scale=2.0)
        close(bits(g_act), act, scale=4.0)
        close(bits(g_out), want, scale=4.0)
    finally:
        eng.close()
