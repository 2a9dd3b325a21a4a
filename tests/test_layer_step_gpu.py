"""Two whole talker decoder layers at decode time, through the library's entry points in the reference's
decode_device order (17.cu:17247-17397), against the same chain built from the oracle's bit-faithful operators.
Errors of the fp32-accumulating kernels compound over the chain, so the bound is twice the single-operator one."""
import numpy as np
import pytest

from oracle import qm_oracle as oracle
import scenario

pytestmark = pytest.mark.gpu


def test_two_layer_decode_step_matches_oracle_chain(qm):
    import torch

    hidden, inter, layers, hq, hkv, d = 256, 512, 2, 16, 8, 128
    lengths = [70, 5, 129]
    b = len(lengths)
    tb = scenario._bf16_tensor
    rng_seed = 500
    x0 = oracle.normal_bf16(rng_seed, (b, hidden))
    weights = []
    for layer in range(layers):
        s = rng_seed + 10 * (layer + 1)
        weights.append({
            "in_norm": oracle.f32_to_bf16(1.0 + 0.1 * oracle.bf16_to_f32(oracle.normal_bf16(s, (hidden,)))),
            "post_norm": oracle.f32_to_bf16(1.0 + 0.1 * oracle.bf16_to_f32(oracle.normal_bf16(s + 1, (hidden,)))),
            "q": oracle.scaled_normal_bf16(s + 2, (hq * d, hidden), 0.06), "k": oracle.scaled_normal_bf16(s + 3, (hkv * d, hidden), 0.06),
            "v": oracle.scaled_normal_bf16(s + 4, (hkv * d, hidden), 0.06), "o": oracle.scaled_normal_bf16(s + 5, (hidden, hq * d), 0.02),
            "gate": oracle.scaled_normal_bf16(s + 6, (inter, hidden), 0.06), "up": oracle.scaled_normal_bf16(s + 7, (inter, hidden), 0.06),
            "down": oracle.scaled_normal_bf16(s + 8, (hidden, inter), 0.04),
        })
    # one scenario per layer supplies the pre-existing cache content, page table and q/k norm weights
    scs = [scenario.DecodeScenario(seed=60 + layer, lengths=lengths, random_weights=True) for layer in range(layers)]
    sc0 = scs[0]

    # ---- oracle chain
    cur = x0
    for layer in range(layers):
        w, sc = weights[layer], scs[layer]
        normed = oracle.rmsnorm(cur, w["in_norm"])
        q = oracle.linear(normed, w["q"]).reshape(b, hq, d)
        k = oracle.linear(normed, w["k"]).reshape(b, hkv, d)
        v = oracle.linear(normed, w["v"]).reshape(b, hkv, d)
        ctx = np.empty((b, hq, d), dtype=np.uint16)
        for s in range(b):
            pos = int(sc.lengths[s])
            kc, vc = sc.key_caches[s].copy(), sc.value_caches[s].copy()
            qr = oracle.append(q[s:s + 1], k[s:s + 1], v[s:s + 1], sc.q_w, sc.k_w, sc.cos[pos:pos + 1], sc.sin[pos:pos + 1], pos, kc, vc)
            ctx[s] = oracle.decode_attention(qr, [kc], [vc], [pos + 1], mode="ref")[0]
        attn = oracle.linear(ctx.reshape(b, hq * d), w["o"])
        residual, post = oracle.add_postnorm(cur, attn, w["post_norm"])
        act = oracle.gate_up_swiglu(post, w["gate"], w["up"])
        cur = oracle.linear(act, w["down"], residual=residual)
    want = cur

    # ---- the library
    eng = qm.TalkerAttention(layers=layers, num_pages=sc0.num_pages, max_positions=sc0.max_pos)
    try:
        for layer in range(layers):
            kp, vp = scs[layer].pools()
            kview, vview = eng.pool_view(layer)
            kview.copy_(tb(torch, kp))
            vview.copy_(tb(torch, vp))
        positions = torch.from_numpy(sc0.lengths).cuda()
        cur_d = tb(torch, x0)
        for layer in range(layers):
            w, sc = weights[layer], scs[layer]
            table = torch.from_numpy(np.maximum(sc.page_table, 0)).cuda()
            normed = eng.launch_rmsnorm(cur_d, tb(torch, w["in_norm"]))
            q, k, v = eng.launch_qkv_m1(normed, tb(torch, w["q"]), tb(torch, w["k"]), tb(torch, w["v"]))
            ctx = eng.decode_step(layer, q.view(b, hq, d), k.view(b, hkv, d), v.view(b, hkv, d), tb(torch, sc.q_w),
                                  tb(torch, sc.k_w), positions, table)
            attn = eng.launch_linear_m1(ctx.view(b, hq * d), tb(torch, w["o"]))
            residual, post = eng.launch_add_postnorm_m1(cur_d, attn, tb(torch, w["post_norm"]))
            act = eng.launch_gate_up_swiglu_m1(post, tb(torch, w["gate"]), tb(torch, w["up"]))
            cur_d = eng.launch_linear_m1(act, tb(torch, w["down"]), residual=residual)
        torch.cuda.synchronize()
        assert eng.status() == 0
        got = scenario._bits(cur_d)
    finally:
        eng.close()
    m = oracle.error_metrics(oracle.bf16_to_f32(got), oracle.bf16_to_f32(want))
    print("two-layer chain", m)
    assert m["max_abs"] <= 8e-2 and m["mean_rel"] <= 2e-2, m
