"""The Gated-DeltaNet decode step and the attention output gate on the GPU (ribn_b200_op_gdn_step,
ribn_b200_op_attention_gate) against the CPU oracle (oracle/gdn.c), on the fixtures and with the tolerances of
the reference's device tests (crates/nvidia/tests/cuda_reference.rs:1002-1056 gates 1e-5, 2144-2201 convolution
1e-4, 2282-2395 state update 1e-2) and at the pinned geometry (16 key heads, 48 value heads, width 128)."""
import numpy as np
import pytest

from oracle import binding as orc
from tests.test_gdn_oracle import fixture_values

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built_library):
    from ribn_b200 import ops as module
    return module


def _case(rng, members, k_heads, v_heads, hd):
    channels, inner = (2 * k_heads + v_heads) * hd, v_heads * hd
    weights = dict(dt_bias=rng.normal(0, 0.3, v_heads), a=-np.exp(rng.normal(0, 0.3, v_heads)),
                   conv_weight=rng.normal(0, 0.5, (channels, 4)), norm_weight=rng.normal(1, 0.1, hd))
    rows = dict(qkv=rng.normal(0, 1, (members, channels)), z=rng.normal(0, 1, (members, inner)),
                beta_raw=rng.normal(0, 1, (members, v_heads)), alpha_raw=rng.normal(0, 1, (members, v_heads)))
    conv = rng.normal(0, 1, (members, channels, 3)).astype(np.float32)
    state = rng.normal(0, 0.05, (members, v_heads, hd, hd)).astype(np.float32)
    return weights, rows, conv, state


@pytest.mark.parametrize("members,k_heads,v_heads,hd", [(1, 16, 48, 128), (3, 4, 8, 64), (5, 2, 2, 128)],
                         ids=["pinned-geometry", "three-sequences-width-64", "five-sequences-untiled"])
def test_gdn_step_matches_the_oracle_over_three_tokens(ops, members, k_heads, v_heads, hd):
    rng = np.random.default_rng(100 + members)
    weights, _, conv, state = _case(rng, members, k_heads, v_heads, hd)
    ref_conv, ref_state = conv.copy(), state.copy()
    for step in range(3):   # the second and third tokens run on the state the device itself left behind
        _, rows, _, _ = _case(rng, members, k_heads, v_heads, hd)
        got = ops.gdn_step(conv_state=conv, state=state, k_heads=k_heads, v_heads=v_heads, head_dim=hd, l2_eps=1e-6,
                           norm_eps=1e-6, **rows, **weights)
        for m in range(members):
            want = orc.gdn_step(conv_state=ref_conv[m], state=ref_state[m], k_heads=k_heads, v_heads=v_heads, head_dim=hd,
                                l2_eps=1e-6, norm_eps=1e-6, **{k: v[m] for k, v in rows.items()}, **weights)
            assert np.max(np.abs(got["decay"][m] - want["decay"])) < 1e-5 and np.max(np.abs(got["beta"][m] - want["beta"])) < 1e-5
            assert np.max(np.abs(got["conv_act"][m] - want["conv_act"])) < 1e-4
            assert np.array_equal(got["conv_state"][m].reshape(-1), want["conv_state"].reshape(-1))   # a shift: exact
            assert np.max(np.abs(got["attn_out"][m] - want["attn_out"])) < 1e-4, (step, m)
            assert np.max(np.abs(got["state"][m].reshape(-1) - want["state"].reshape(-1))) < 1e-5
            assert np.max(np.abs(got["out"][m] - want["out"])) < 1e-3, (step, m)
            ref_conv[m], ref_state[m] = want["conv_state"].reshape(ref_conv[m].shape), want["state"].reshape(ref_state[m].shape)
        conv, state = got["conv_state"], got["state"]


def test_gdn_step_is_independent_of_the_batch(ops):
    """A sequence's step gives the same bits alone and among others (sums have a fixed order)."""
    rng = np.random.default_rng(7)
    weights, rows, conv, state = _case(rng, 4, 4, 8, 128)
    batch = ops.gdn_step(conv_state=conv, state=state, k_heads=4, v_heads=8, head_dim=128, l2_eps=1e-6, norm_eps=1e-6, **rows, **weights)
    alone = ops.gdn_step(conv_state=conv[2:3], state=state[2:3], k_heads=4, v_heads=8, head_dim=128, l2_eps=1e-6, norm_eps=1e-6,
                         **{k: v[2:3] for k, v in rows.items()}, **weights)
    assert np.array_equal(batch["out"][2], alone["out"][0]) and np.array_equal(batch["state"][2], alone["state"][0])


def test_state_update_on_the_reference_fixture(ops):
    """cuda_reference.rs:2282-2395: unnormalised fixture vectors at 48 / 16 / 128, held to its 1e-2 (relative to the
    size of the sums).  The step normalises q and k itself, so the fixture's vectors enter as convolution outputs
    whose normalised form the oracle computes the same way."""
    v_heads, k_heads, hd = 48, 16, 128
    channels = (2 * k_heads + v_heads) * hd
    matrix, lcg = fixture_values(99, v_heads * hd * hd)
    matrix = (matrix * np.float32(0.05)).astype(np.float32).reshape(1, v_heads, hd, hd)
    qkv, lcg = fixture_values(lcg, channels)
    history, lcg = fixture_values(lcg, channels * 3)
    conv_weight = np.zeros((channels, 4), np.float32); conv_weight[:, 3] = 1.0     # the convolution passes the new token through
    common = dict(z=np.ones((1, v_heads * hd), np.float32), beta_raw=np.linspace(-2, 2, v_heads, dtype=np.float32)[None],
                  alpha_raw=np.linspace(-1, 1, v_heads, dtype=np.float32)[None], dt_bias=np.zeros(v_heads, np.float32),
                  a=-np.ones(v_heads, np.float32), conv_weight=conv_weight, norm_weight=np.ones(hd, np.float32))
    got = ops.gdn_step(qkv=qkv[None], conv_state=history.reshape(1, channels, 3), state=matrix, k_heads=k_heads, v_heads=v_heads,
                       head_dim=hd, l2_eps=1e-5, norm_eps=1e-6, **common)
    want = orc.gdn_step(qkv=qkv, conv_state=history.reshape(channels, 3), state=matrix[0], k_heads=k_heads, v_heads=v_heads,
                        head_dim=hd, l2_eps=1e-5, norm_eps=1e-6, **{k: (v[0] if v.ndim == 2 and k in ("z", "beta_raw", "alpha_raw") else v) for k, v in common.items()})
    scale = max(1.0, float(np.max(np.abs(want["attn_out"]))))
    assert np.max(np.abs(got["attn_out"][0] - want["attn_out"])) < 1e-2 * scale
    assert np.max(np.abs(got["state"][0].reshape(-1) - want["state"].reshape(-1))) < 1e-2


def test_attention_gate_matches_the_oracle(ops):
    rng = np.random.default_rng(3)
    rows, heads, width = 5, 24, 256
    attn = rng.normal(0, 1, (rows, heads * width)).astype(np.float32)
    q_gate = rng.normal(0, 3, (rows, heads * 2 * width)).astype(np.float32)
    got = ops.attention_gate(attn, q_gate, heads, width)
    want = orc.attention_gate(attn, q_gate, rows, heads, width)
    assert np.max(np.abs(got - want.reshape(got.shape))) < 1e-6


def test_several_tokens_in_one_call_equal_single_steps_bit_for_bit(ops):
    """The prefill form: five consecutive tokens of two sequences in one call (the state stays in registers) against
    the same tokens as five single-step calls, and the last token against the oracle."""
    rng = np.random.default_rng(21)
    members, tokens, k_heads, v_heads, hd = 2, 5, 4, 8, 128
    weights, _, conv, state = _case(rng, members, k_heads, v_heads, hd)
    steps = [_case(rng, members, k_heads, v_heads, hd)[1] for _ in range(tokens)]
    stacked = {k: np.stack([steps[t][k] for t in range(tokens)], axis=1).reshape(members * tokens, -1) for k in steps[0]}
    chunk = ops.gdn_step(conv_state=conv, state=state, k_heads=k_heads, v_heads=v_heads, head_dim=hd, l2_eps=1e-6, norm_eps=1e-6,
                         tokens=tokens, **stacked, **weights)
    c, s_, ref_c, ref_s = conv, state, conv.copy(), state.copy()
    for t in range(tokens):
        one = ops.gdn_step(conv_state=c, state=s_, k_heads=k_heads, v_heads=v_heads, head_dim=hd, l2_eps=1e-6, norm_eps=1e-6,
                           **steps[t], **weights)
        for m in range(members):
            assert np.array_equal(chunk["out"][m * tokens + t], one["out"][m])
            assert np.array_equal(chunk["conv_act"][m * tokens + t], one["conv_act"][m])
            want = orc.gdn_step(conv_state=ref_c[m], state=ref_s[m], k_heads=k_heads, v_heads=v_heads, head_dim=hd, l2_eps=1e-6,
                                norm_eps=1e-6, **{k: v[m] for k, v in steps[t].items()}, **weights)
            ref_c[m], ref_s[m] = want["conv_state"].reshape(ref_c[m].shape), want["state"].reshape(ref_s[m].shape)
            if t == tokens - 1:
                assert np.max(np.abs(chunk["out"][m * tokens + t] - want["out"])) < 1e-3
        c, s_ = one["conv_state"], one["state"]
    assert np.array_equal(chunk["state"], s_) and np.array_equal(chunk["conv_state"], c)
