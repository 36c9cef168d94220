"""Dequant-fused GEMV on the GPU against the CPU oracle: the reference's
fixtures and tolerances (crates/nvidia/tests/cuda_reference.rs:690-846, 4842-4880,
5172-5278), seeded N(0, 0.02) checkpoints of BASELINE shapes, ragged row counts,
and batch-vs-single bit equality.  variant 0 = tensor-core kernels over the
tile-major repack, variant 1 = the plain one-warp-per-row kernels, variant 2 = the
batched tensor-core kernel (3..64 members per launch, one activation scale per member)."""
import numpy as np
import pytest

from oracle import binding as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built_library):
    from ribn_b200 import ops as o
    orc.set_threads(8)
    return o


@pytest.mark.parametrize("variant", [1, 0])
@pytest.mark.parametrize("kind", [H.Q4_K, H.Q6_K])
def test_reference_fixture_within_1e3(ops, kind, variant):
    enc = H.fixture(kind)            # [512, 2] fixture: 2 rows x 2 blocks
    x = H.fixture_input(512)
    want = orc.gemv(kind, enc, 512, 2, x)
    got = ops.gemv(kind, enc, 2, 512, x, variant=variant)
    assert np.max(np.abs(got - want)) < 1e-3


def test_q8_0_fixture_reference_kernel(ops):
    enc = H.fixture(H.Q8_0)          # 6 blocks: 2 rows x 96
    x = H.fixture_input(96)
    assert np.max(np.abs(ops.gemv(H.Q8_0, enc, 2, 96, x, variant=1) - orc.gemv(H.Q8_0, enc, 96, 2, x))) < 1e-3


@pytest.mark.parametrize("variant", [1, 0])
@pytest.mark.parametrize("kind", [H.Q8_0, H.Q4_K, H.Q6_K])
@pytest.mark.parametrize("rows,cols", [(1, 256), (5, 512), (40, 1024), (256, 4096), (128, 12288)])
def test_quantised_normal_weights(ops, kind, rows, cols, variant):
    rng = np.random.default_rng(rows * 7 + cols + kind)
    enc = H.quantize(kind, rng.normal(0, 0.02, size=(rows, cols)).astype(np.float32))
    x = rng.normal(0, 1, cols).astype(np.float32)
    want = orc.gemv(kind, enc, cols, rows, x)
    got = ops.gemv(kind, enc, rows, cols, x, variant=variant)
    scale = float(np.max(np.abs(want))) + 1e-6
    assert np.max(np.abs(got - want)) < 1e-3
    assert np.max(np.abs(got - want)) / scale < 2e-5


@pytest.mark.parametrize("kind", [H.Q8_0, H.Q4_K, H.Q6_K])
def test_random_bytes_blocks_exercise_every_bit_field(ops, kind):
    # uniform random bytes: all scale/min/high-bit fields populated; f16 scales kept small and finite
    rng = np.random.default_rng(kind + 1)
    elems, size = H.BLOCK[kind]
    rows, cols = 48, 512
    blocks = rng.integers(0, 256, size=(rows * cols // elems, size), dtype=np.uint8)
    for off in ([0] if kind == H.Q8_0 else [0, 2] if kind == H.Q4_K else [208]):
        blocks[:, off + 1] = (blocks[:, off + 1] & 0x83) | 0x10  # |d| in [2^-11, 2^-8)
    x = rng.normal(0, 1, cols).astype(np.float32)
    want = orc.gemv(kind, blocks, cols, rows, x)
    for variant in (1, 0):
        got = ops.gemv(kind, blocks, rows, cols, x, variant=variant)
        assert np.max(np.abs(got - want)) / (np.max(np.abs(want)) + 1e-9) < 2e-5


@pytest.mark.parametrize("kind", [H.Q8_0, H.Q4_K, H.Q6_K])
def test_batch_rows_equal_single_row_bits(ops, kind):
    # crates/nvidia/tests/cuda_reference.rs:5172-5278: members use input (i + 7m) % 17
    rng = np.random.default_rng(kind)
    rows, cols = 64, 1024
    enc = H.quantize(kind, rng.normal(0, 0.02, size=(rows, cols)).astype(np.float32))
    xs = np.stack([H.fixture_input(cols, m) * np.float32(1 + m) for m in range(7)])
    for variant in (0, 1):
        batch = ops.gemv(kind, enc, rows, cols, xs, variant=variant)
        for m in range(7):
            single = ops.gemv(kind, enc, rows, cols, xs[m], variant=variant)
            assert np.array_equal(batch[m].view(np.uint32), single.view(np.uint32))
        want = np.stack([orc.gemv(kind, enc, cols, rows, xs[m]) for m in range(7)])
        assert np.max(np.abs(batch - want)) < 1e-3


def test_activation_range_extremes(ops):
    # per-vector power-of-two scaling keeps huge and tiny activations inside binary16 range
    rng = np.random.default_rng(8)
    enc = H.quantize(H.Q4_K, rng.normal(0, 0.02, size=(32, 512)).astype(np.float32))
    for mag in (1e-6, 1.0, 3e5, 1e9):
        x = (rng.normal(0, 1, 512) * mag).astype(np.float32)
        want = orc.gemv(H.Q4_K, enc, 512, 32, x)
        got = ops.gemv(H.Q4_K, enc, 32, 512, x, variant=0)
        assert np.max(np.abs(got - want)) / np.max(np.abs(want)) < 2e-5
    zero = ops.gemv(H.Q4_K, enc, 32, 512, np.zeros(512, np.float32), variant=0)
    assert np.all(zero == 0.0)


def test_full_size_projection_fast_equals_reference_kernel_and_is_linear(ops):
    # Qwen3-8B ffn_down shape (12288 -> 4096, Q6_K) and q shape (4096 -> 4096, Q4_K):
    # size-independent properties at BASELINE's full sizes.
    rng = np.random.default_rng(21)
    for kind, rows, cols in ((H.Q6_K, 4096, 12288), (H.Q4_K, 4096, 4096)):
        elems, size = H.BLOCK[kind]
        blocks = rng.integers(0, 256, size=(rows * cols // elems, size), dtype=np.uint8)
        for off in ([0, 2] if kind == H.Q4_K else [208]):
            blocks[:, off + 1] = (blocks[:, off + 1] & 0x83) | 0x10
        x1 = rng.normal(0, 1, cols).astype(np.float32)
        x2 = rng.normal(0, 1, cols).astype(np.float32)
        fast = ops.gemv(kind, blocks, rows, cols, np.stack([x1, x2, x1 + x2]), variant=0)
        ref = ops.gemv(kind, blocks, rows, cols, np.stack([x1, x2]), variant=1)
        scale = np.max(np.abs(ref))
        assert np.max(np.abs(fast[:2] - ref)) / scale < 2e-5
        assert np.max(np.abs(fast[2] - (fast[0] + fast[1]))) / scale < 2e-5
        spot = rng.integers(0, rows, 8)
        for r in spot:
            row_bytes = blocks.reshape(rows, -1)[r]
            assert abs(orc.gemv(kind, row_bytes, cols, 1, x1)[0] - fast[0][r]) / scale < 2e-5


@pytest.mark.parametrize("kind", [H.Q8_0, H.Q4_K, H.Q6_K])
@pytest.mark.parametrize("rows,cols,members", [(1, 256, 1), (5, 512, 3), (70, 1024, 9), (256, 4096, 64), (96, 12288, 17),
                                               (40, 768, 131)])
def test_batched_kernel_against_oracle(ops, kind, rows, cols, members):
    rng = np.random.default_rng(rows * 11 + cols + kind + members)
    enc = H.quantize(kind, rng.normal(0, 0.02, size=(rows, cols)).astype(np.float32))
    xs = (rng.normal(0, 1, size=(members, cols)) * rng.uniform(0.1, 10, size=(members, 1))).astype(np.float32)
    got = ops.gemv(kind, enc, rows, cols, xs, variant=2)
    want = np.stack([orc.gemv(kind, enc, cols, rows, xs[m]) for m in range(members)])
    for m in range(members):
        scale = float(np.max(np.abs(want[m]))) + 1e-6
        assert np.max(np.abs(got[m] - want[m])) / scale < 2e-5, m


@pytest.mark.parametrize("kind", [H.Q8_0, H.Q4_K, H.Q6_K])
def test_batched_kernel_random_bytes_and_member_independence(ops, kind):
    rng = np.random.default_rng(kind + 77)
    elems, size = H.BLOCK[kind]
    rows, cols = 80, 1024
    blocks = rng.integers(0, 256, size=(rows * cols // elems, size), dtype=np.uint8)
    for off in ([0] if kind == H.Q8_0 else [0, 2] if kind == H.Q4_K else [208]):
        blocks[:, off + 1] = (blocks[:, off + 1] & 0x83) | 0x10
    xs = rng.normal(0, 1, size=(20, cols)).astype(np.float32)
    got = ops.gemv(kind, blocks, rows, cols, xs, variant=2)
    want = np.stack([orc.gemv(kind, blocks, cols, rows, xs[m]) for m in range(20)])
    assert np.max(np.abs(got - want)) / np.max(np.abs(want)) < 2e-5
    # a member's result does not depend on what it is batched with, nor on its place in the batch
    alone = ops.gemv(kind, blocks, rows, cols, xs[[5, 0, 13]], variant=2)
    assert np.array_equal(alone.view(np.uint32), got[[5, 0, 13]].view(np.uint32))
    zero = ops.gemv(kind, blocks, rows, cols, np.zeros((3, cols), np.float32), variant=2)
    assert np.all(zero == 0.0)


@pytest.mark.parametrize("variant", [3, 4])
@pytest.mark.parametrize("kind", [H.Q4_K, H.Q6_K, H.Q8_0])
@pytest.mark.parametrize("rows,cols,members", [(16, 256, 1), (130, 512, 5), (256, 1024, 64), (300, 4096, 128),
                                               (128, 12288, 33), (64, 768, 150), (272, 1024, 200), (144, 12288, 128)])
def test_tensor_memory_kernels_against_oracle(ops, kind, rows, cols, members, variant):
    # tcgen05 kernels.  K-quant form (variant 3 on Q4_K / Q6_K; 128 members and more run their whole groups of 64 in
    # one launch whose work items take two groups each, 200 members = a pair, an odd group and 8 more rows): the
    # tensor core multiplies the blocks'
    # exact integers and the F32 scales are applied per 256 inputs with round-to-nearest FMAs.
    # Decode-and-split form (variant 4, and Q8_0): weights and activations enter as binary16 hi + lo
    # pairs and the whole K is accumulated in tensor memory, whose F32 accumulation is not
    # round-to-nearest: the error grows with K (about 3e-5 of the largest output at K = 12288).
    # The reference's own tolerance for this operator is 1e-3 absolute (cuda_reference.rs:690-846).
    if variant == 4 and kind == H.Q8_0:
        pytest.skip("variant 3 already takes the decode-and-split form for Q8_0")
    rng = np.random.default_rng(rows * 13 + cols + kind + members)
    enc = H.quantize(kind, rng.normal(0, 0.02, size=(rows, cols)).astype(np.float32))
    xs = (rng.normal(0, 1, size=(members, cols)) * rng.uniform(0.01, 100, size=(members, 1))).astype(np.float32)
    got = ops.gemv(kind, enc, rows, cols, xs, variant=variant)
    want = np.stack([orc.gemv(kind, enc, cols, rows, xs[m]) for m in range(members)])
    tolerance = 2e-5 if (variant == 3 and kind != H.Q8_0) else 1e-4
    for m in range(members):
        scale = float(np.max(np.abs(want[m]))) + 1e-6
        assert np.max(np.abs(got[m] - want[m])) / scale < tolerance, m


@pytest.mark.parametrize("variant", [3, 4])
@pytest.mark.parametrize("kind", [H.Q4_K, H.Q6_K, H.Q8_0])
def test_tensor_memory_kernels_random_bytes_and_member_independence(ops, kind, variant):
    rng = np.random.default_rng(kind + 177)
    elems, size = H.BLOCK[kind]
    rows, cols = 144, 1024
    blocks = rng.integers(0, 256, size=(rows * cols // elems, size), dtype=np.uint8)
    for off in ([0] if kind == H.Q8_0 else [0, 2] if kind == H.Q4_K else [208]):
        blocks[:, off + 1] = (blocks[:, off + 1] & 0x83) | 0x10
    xs = rng.normal(0, 1, size=(20, cols)).astype(np.float32)
    got = ops.gemv(kind, blocks, rows, cols, xs, variant=variant)
    want = np.stack([orc.gemv(kind, blocks, cols, rows, xs[m]) for m in range(20)])
    assert np.max(np.abs(got - want)) / np.max(np.abs(want)) < 1e-4
    alone = ops.gemv(kind, blocks, rows, cols, xs[[5, 0, 13]], variant=variant)
    assert np.array_equal(alone.view(np.uint32), got[[5, 0, 13]].view(np.uint32))
    zero = ops.gemv(kind, blocks, rows, cols, np.zeros((3, cols), np.float32), variant=variant)
    assert np.all(zero == 0.0)
    huge = ops.gemv(kind, blocks, rows, cols, xs[:3] * np.float32(1e9), variant=variant)
    assert np.max(np.abs(huge / np.float32(1e9) - want[:3])) / np.max(np.abs(want)) < 1e-4


@pytest.mark.parametrize("kind", [H.Q4_K, H.Q6_K])
@pytest.mark.parametrize("rows,cols,members", [(19200, 512, 256), (37888, 256, 197)], ids=["two-pairs", "pair-odd-group-and-rest"])
def test_tensor_memory_pair_kernel_against_oracle(ops, kind, rows, cols, members):
    """Enough output rows that the launcher gives each work item two row groups (one conversion of a weight stage
    per pair): four whole groups as two pairs; three whole groups as a pair plus an odd group, and five more rows.
    Sampled members of every group against the oracle, and bit equality with the same rows run alone."""
    rng = np.random.default_rng(rows + members + kind)
    enc = H.quantize(kind, rng.normal(0, 0.02, size=(rows, cols)).astype(np.float32))
    xs = (rng.normal(0, 1, size=(members, cols)) * rng.uniform(0.01, 100, size=(members, 1))).astype(np.float32)
    got = ops.gemv(kind, enc, rows, cols, xs, variant=3)
    picks = sorted(set([0, 31, 63, 64, 100, 127, 128, 191, members - 1]))
    for m in picks:
        want = orc.gemv(kind, enc, cols, rows, xs[m])
        scale = float(np.max(np.abs(want))) + 1e-6
        assert np.max(np.abs(got[m] - want)) / scale < 2e-5, m
    alone = ops.gemv(kind, enc, rows, cols, xs[[70, 130]], variant=3)   # the single-group kernel
    assert np.array_equal(alone.view(np.uint32), got[[70, 130]].view(np.uint32))


@pytest.mark.parametrize("kind", [H.Q4_K, H.Q6_K])
@pytest.mark.parametrize("rows,cols,members", [
    (200, 256, 3), (1000, 512, 17), (4096, 4096, 64), (19200, 512, 256), (37888, 256, 197), (640, 2048, 130),
], ids=["one-k-tile-ragged-unit", "ragged-rows", "k-slices", "two-pairs", "pair-odd-group-and-rest", "pair-and-rest-few-units"])
def test_operand_cache_gemm_changes_no_bit(ops, kind, rows, cols, members):
    """The K-quant GEMM over operands converted once (variant 5: stages are copied, not converted) gives the bits of
    the converting kernels (variant 3) at every shape class: a unit with missing row tiles, one k tile, split K,
    groups in pairs with an odd group and a partial last group.  One member also against the oracle."""
    rng = np.random.default_rng(rows * 7 + members + kind)
    enc = H.quantize(kind, rng.normal(0, 0.02, size=(rows, cols)).astype(np.float32))
    xs = (rng.normal(0, 1, size=(members, cols)) * rng.uniform(0.01, 100, size=(members, 1))).astype(np.float32)
    converting = ops.gemv(kind, enc, rows, cols, xs, variant=3)
    cached = ops.gemv(kind, enc, rows, cols, xs, variant=5)
    assert np.array_equal(cached.view(np.uint32), converting.view(np.uint32))
    m = members - 1
    want = orc.gemv(kind, enc, cols, rows, xs[m])
    assert np.max(np.abs(cached[m] - want)) / (float(np.max(np.abs(want))) + 1e-6) < 2e-5


def test_operand_cache_refuses_other_types(ops):
    rng = np.random.default_rng(5)
    enc = H.quantize(H.Q8_0, rng.normal(0, 0.02, size=(128, 256)).astype(np.float32))
    with pytest.raises(RuntimeError):
        ops.gemv(H.Q8_0, enc, 128, 256, np.ones((4, 256), np.float32), variant=5)
