"""The Gated-DeltaNet oracle (oracle/gdn.c) against an independent float64 evaluation of the reference's host
equations (crates/nvidia/src/qwen_reference.rs:42-141, 202-278) on the fixtures of the reference's own device
tests (crates/nvidia/tests/cuda_reference.rs:1002-1056, 2144-2201, 2203-2270, 2282-2395), with those tests'
tolerances.  The fixture generator is the reference's fixture_quantized_f32 (cuda_reference.rs:1603-1607)."""
import numpy as np

from oracle import binding as orc


def fixture_values(state: int, count: int):
    """fixture_quantized_f32: an LCG whose bits 16..21 pick one of 64 multiples of 0.125 from -4."""
    out = np.empty(count, dtype=np.float32)
    for i in range(count):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = np.float32(((state >> 16) & 0x3F) * 0.125 - 4.0)
    return out, state


def test_scalar_gate_fixture():
    heads = 16
    idx = np.arange(heads, dtype=np.float32)
    alpha, beta_raw = (-0.5 + idx * np.float32(0.07)).astype(np.float32), (idx * np.float32(0.11) - np.float32(0.8)).astype(np.float32)
    dt_bias, a = (-0.3 + idx * np.float32(0.05)).astype(np.float32), (-1.0 - idx * np.float32(0.1)).astype(np.float32)
    decay, beta = orc.gdn_scalar_gate(alpha, beta_raw, dt_bias, a)
    arg = alpha.astype(np.float64) + dt_bias
    want_decay = np.exp(a.astype(np.float64) * np.log1p(np.exp(arg)))
    want_beta = 1.0 / (1.0 + np.exp(-beta_raw.astype(np.float64)))
    assert np.max(np.abs(decay - want_decay)) < 1e-5 and np.max(np.abs(beta - want_beta)) < 1e-5
    # the large-input shortcut of softplus (qwen_reference.rs:51-58)
    decay, _ = orc.gdn_scalar_gate([25.0], [0.0], [0.0], [-0.01])
    assert abs(float(decay[0]) - float(np.exp(-0.25))) < 1e-6


def test_conv_silu_fixture():
    channels = 512
    x, state = fixture_values(777, channels)
    weight, state = fixture_values(state, channels * 4)
    history, state = fixture_values(state, channels * 3)
    raw, act, advanced = orc.gdn_conv_silu(x, weight, history)
    h, w = history.reshape(channels, 3).astype(np.float64), weight.reshape(channels, 4).astype(np.float64)
    want = h[:, 0] * w[:, 0] + h[:, 1] * w[:, 1] + h[:, 2] * w[:, 2] + x.astype(np.float64) * w[:, 3]
    assert np.max(np.abs(raw - want)) < 1e-4
    assert np.max(np.abs(act - want / (1.0 + np.exp(-want)))) < 1e-4
    adv = advanced.reshape(channels, 3)
    assert np.array_equal(adv[:, 0], history.reshape(channels, 3)[:, 1]) and np.array_equal(adv[:, 1], history.reshape(channels, 3)[:, 2])
    assert np.array_equal(adv[:, 2], x)


def test_l2_norm_heads_fixture_and_eps_floor():
    heads, hd, eps = 16, 128, 1e-5
    x, _ = fixture_values(4242, heads * hd)
    got = orc.l2_norm_heads(x, heads, hd, eps).reshape(heads, hd)
    v = x.reshape(heads, hd).astype(np.float64)
    want = v / np.maximum(np.sqrt(np.sum(v * v, axis=1, keepdims=True)), eps)
    assert np.max(np.abs(got - want)) < 1e-4
    zero = orc.l2_norm_heads(np.zeros(hd, np.float32), 1, hd, eps)   # 1 / max(0, eps): stays zero, no NaN
    assert np.all(zero == 0.0)


def state_update_f64(matrix, q, k, conv, decay, beta, v_heads, k_heads, hd, v_offset):
    m = matrix.reshape(v_heads, hd, hd).astype(np.float64).copy()
    out = np.empty((v_heads, hd))
    for h in range(v_heads):
        qh, kh = q.reshape(k_heads, hd)[h % k_heads].astype(np.float64), k.reshape(k_heads, hd)[h % k_heads].astype(np.float64)
        v = conv[v_offset + h * hd: v_offset + (h + 1) * hd].astype(np.float64)
        m[h] *= float(decay[h])
        d = (v - m[h].T @ kh) * float(beta[h])
        m[h] += np.outer(kh, d)
        out[h] = (m[h].T @ qh) / np.sqrt(hd)
    return out.reshape(-1), m.reshape(-1)


def test_state_update_fixture_at_the_pinned_geometry():
    v_heads, k_heads, hd, v_offset = 48, 16, 128, 4096
    matrix, state = fixture_values(99, v_heads * hd * hd)
    matrix = (matrix * np.float32(0.05)).astype(np.float32)
    conv, state = fixture_values(state, v_offset + v_heads * hd)
    q, state = fixture_values(state, k_heads * hd)
    k, state = fixture_values(state, k_heads * hd)
    decay = (np.arange(v_heads, dtype=np.float32) * np.float32(0.01) + np.float32(0.5)).astype(np.float32)
    beta = (np.arange(v_heads, dtype=np.float32) * np.float32(0.005) + np.float32(0.1)).astype(np.float32)
    out, updated = orc.gdn_state_update(matrix, q, k, conv, decay, beta, v_heads, k_heads, hd, v_offset)
    want_out, want_matrix = state_update_f64(matrix, q, k, conv, decay, beta, v_heads, k_heads, hd, v_offset)
    # unnormalised fixture vectors make sums of order 1e4: the reference's 1e-2 is an absolute bound there
    assert np.max(np.abs(out - want_out)) < 1e-2 * max(1.0, float(np.max(np.abs(want_out))) / 1e2)
    assert np.max(np.abs(updated - want_matrix)) < 1e-2 * max(1.0, float(np.max(np.abs(want_matrix))) / 1e2)


def test_gated_norm_and_attention_gate():
    heads, hd, eps = 48, 128, 1e-6
    rng = np.random.default_rng(5)
    o, z = rng.normal(0, 1, heads * hd).astype(np.float32), rng.normal(0, 2, heads * hd).astype(np.float32)
    norm = rng.normal(1, 0.2, hd).astype(np.float32)
    got = orc.gdn_gated_norm(o, z, norm, heads, hd, eps).reshape(heads, hd)
    o64, z64 = o.reshape(heads, hd).astype(np.float64), z.reshape(heads, hd).astype(np.float64)
    want = o64 / np.sqrt(np.mean(o64 * o64, axis=1, keepdims=True) + eps) * norm * (z64 / (1.0 + np.exp(-z64)))
    assert np.max(np.abs(got - want)) < 1e-5
    rows, qh, width = 3, 24, 256
    attn = rng.normal(0, 1, (rows, qh, width)).astype(np.float32)
    q_gate = rng.normal(0, 2, (rows, qh, 2 * width)).astype(np.float32)
    gated = orc.attention_gate(attn, q_gate, rows, qh, width).reshape(rows, qh, width)
    want = attn.astype(np.float64) / (1.0 + np.exp(-q_gate[:, :, width:].astype(np.float64)))
    assert np.max(np.abs(gated - want)) < 1e-6


def test_whole_step_is_the_composition_and_evolves_with_its_state():
    """host_gdn_ar_step behind the projections: the composed step equals its parts, two steps from the same state
    give the same bits, and a second step depends on what the first left behind (cuda_reference.rs:1215-1365)."""
    k_heads, v_heads, hd = 4, 8, 64
    channels, inner = (2 * k_heads + v_heads) * hd, v_heads * hd
    rng = np.random.default_rng(11)
    args = dict(qkv=rng.normal(0, 1, channels), z=rng.normal(0, 1, inner), beta_raw=rng.normal(0, 1, v_heads),
                alpha_raw=rng.normal(0, 1, v_heads), dt_bias=rng.normal(0, 0.3, v_heads), a=-np.exp(rng.normal(0, 0.3, v_heads)),
                conv_weight=rng.normal(0, 0.5, (channels, 4)), norm_weight=rng.normal(1, 0.1, hd))
    conv0, state0 = rng.normal(0, 1, (channels, 3)), rng.normal(0, 0.05, (v_heads, hd, hd))
    one = orc.gdn_step(conv_state=conv0, state=state0, k_heads=k_heads, v_heads=v_heads, head_dim=hd, l2_eps=1e-6, norm_eps=1e-6, **args)
    again = orc.gdn_step(conv_state=conv0, state=state0, k_heads=k_heads, v_heads=v_heads, head_dim=hd, l2_eps=1e-6, norm_eps=1e-6, **args)
    assert np.array_equal(one["out"], again["out"]) and np.array_equal(one["state"], again["state"])
    decay, beta = orc.gdn_scalar_gate(args["alpha_raw"], args["beta_raw"], args["dt_bias"], args["a"])
    _, act, conv1 = orc.gdn_conv_silu(args["qkv"], args["conv_weight"], conv0)
    q = orc.l2_norm_heads(act[: k_heads * hd], k_heads, hd, 1e-6)
    k = orc.l2_norm_heads(act[k_heads * hd: 2 * k_heads * hd], k_heads, hd, 1e-6)
    o, state1 = orc.gdn_state_update(state0, q, k, act, decay, beta, v_heads, k_heads, hd, 2 * k_heads * hd)
    out = orc.gdn_gated_norm(o, args["z"], args["norm_weight"], v_heads, hd, 1e-6)
    assert np.array_equal(one["out"], out) and np.array_equal(one["state"].reshape(-1), state1.reshape(-1))
    assert np.array_equal(one["conv_state"].reshape(-1), conv1.reshape(-1)) and np.array_equal(one["attn_out"], o)
    second = orc.gdn_step(conv_state=one["conv_state"], state=one["state"], k_heads=k_heads, v_heads=v_heads, head_dim=hd,
                          l2_eps=1e-6, norm_eps=1e-6, **args)
    assert not np.array_equal(second["out"], one["out"])
