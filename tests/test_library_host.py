"""CPU-only checks of the CUDA library's host side: it loads, exports every
symbol the header declares, and its tile-major repack feeds the tensor-core
A fragment the integers the raw GGUF blocks hold (emulated in numpy with the
kernel's own masks and shifts).  No device work is issued here."""
import os
import re

import numpy as np
import pytest

from tests import helpers as H

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(built_library):
    import ribn_b200
    from ribn_b200 import _lib
    header = "".join(open(os.path.join(ROOT, "include", name)).read() for name in ("ribn_b200.h", "ribn_b200_gemma.h", "ribn_b200_engine.h"))
    declared = set(re.findall(r"\b(ribn_b200_[a-z0-9_]+)\s*\(", header))
    assert declared, "header declares nothing?"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    handle = ribn_b200.lib()
    for name in declared:
        assert hasattr(handle, name)
    assert b"sm_100a" in handle.ribn_b200_build_info()


def test_python_flag_constants_mirror_the_header():
    """The ctypes mirror's RIBN_B200_FLAG_* values are the header's (a drifted constant would silently set another
    option on the executor)."""
    from ribn_b200 import _lib
    header = open(os.path.join(ROOT, "include", "ribn_b200.h")).read()
    flags = dict(re.findall(r"RIBN_B200_(FLAG_[A-Z0-9_]+)\s*=\s*(\d+)", header))
    assert {"FLAG_KEEP_LOGITS", "FLAG_NO_GRAPH", "FLAG_KV_ON_DEMAND", "FLAG_OPERAND_CACHE"} <= set(flags)
    for name, value in flags.items():
        assert getattr(_lib, name) == int(value), name
    assert len(set(flags.values())) == len(flags)
    for value in flags.values():
        assert int(value) & (int(value) - 1) == 0, "flags are single bits"


C_CLIENT = r"""
#include <stdio.h>
#include <string.h>
#include "ribn_b200.h"
#include "ribn_b200_gemma.h"
#include "ribn_b200_engine.h"
int main(void) {
    char err[256] = {0};
    ribn_b200_engine* e = NULL;
    ribn_b200_engine_config cfg = {2, 4};
    ribn_b200_schedule_policy pol = {64, 16, 1, 8};
    int rc = ribn_b200_engine_create(NULL, &cfg, &pol, &e, err, sizeof(err));
    printf("%s|%d|%s", ribn_b200_build_info(), rc, err);
    return rc == RIBN_B200_ERROR && strstr(err, "null") ? 0 : 1;
}
"""


def test_headers_are_strict_c99_and_a_c_client_links(built_library, tmp_path):
    """The boundary is a C ABI: the three headers compile as pedantic C99 with warnings as errors, and a C program
    links against the library and calls into it (no device work)."""
    import shutil
    import subprocess
    import ribn_b200
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    src, exe = tmp_path / "client.c", tmp_path / "client"
    src.write_text(C_CLIENT)
    libdir = os.path.dirname(ribn_b200.library_path())
    build = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), str(src),
                            "-o", str(exe), ribn_b200.library_path(), f"-Wl,-rpath,{libdir}"], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "sm_100a" in run.stdout and "null argument" in run.stdout


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "ribn_b200")
    for dirpath, _dirs, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f


NIB, TOPBITS = 0x0F0F0F0F, 0x30303030


def _bytes(reg):
    return [(int(reg) >> (8 * i)) & 0xFF for i in range(4)]


def _place32(Q, g, t, kbase, regs):
    """regs = (a0, a1, a2, a3) of mma.m16n8k32 (u8): rows g / g+8, inputs 4t..4t+3 and 16+4t..16+4t+3."""
    for ri, reg in enumerate(regs):
        row = g + (8 if ri & 1 else 0)
        k = kbase + 4 * t + (16 if ri >= 2 else 0)
        for i, b in enumerate(_bytes(reg)):
            Q[row, k + i] = b


def _place16(Q, g, t, kbase, regs):
    """regs = (a0, a1) of mma.m16n8k16 (u8): rows g / g+8, inputs 4t..4t+3."""
    for ri, reg in enumerate(regs):
        for i, b in enumerate(_bytes(reg)):
            Q[g + 8 * ri, kbase + 4 * t + i] = b


def _words(tile, off):
    return np.frombuffer(tile[off:off + 16].tobytes(), dtype="<u4").astype(np.int64)


def emulate_q4k(tile):
    Q = np.zeros((16, 256), dtype=np.int64)
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        for j in range(4):
            x, y, z, w = _words(tile, j * 512 + lane * 16)
            _place32(Q, g, t, 2 * j * 32, (x & NIB, z & NIB, y & NIB, w & NIB))
            _place32(Q, g, t, (2 * j + 1) * 32, ((x >> 4) & NIB, (z >> 4) & NIB, (y >> 4) & NIB, (w >> 4) & NIB))
    return Q


def emulate_q6k(tile):
    Q = np.zeros((16, 256), dtype=np.int64)
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        for c in range(2):
            qh = _words(tile, 2048 + c * 512 + lane * 16)
            for h in range(2):
                la0, lb0, la1, lb1 = _words(tile, (c * 2 + h) * 512 + lane * 16)
                wh0, wh1 = (qh[0], qh[1]) if h == 0 else (qh[2], qh[3])
                for v in range(4):
                    l0, l1 = (lb0, lb1) if v & 1 else (la0, la1)
                    sh = 4 - 2 * v
                    t0 = (wh0 << sh) if sh >= 0 else (wh0 >> -sh)
                    t1 = (wh1 << sh) if sh >= 0 else (wh1 >> -sh)
                    a0 = ((l0 if v < 2 else l0 >> 4) & NIB) | (t0 & TOPBITS)
                    a1 = ((l1 if v < 2 else l1 >> 4) & NIB) | (t1 & TOPBITS)
                    _place16(Q, g, t, (c * 4 + v) * 32 + 16 * h, (a0, a1))
    return Q


def emulate_q8_0(tile):
    Q = np.zeros((16, 256), dtype=np.int64)
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        for b in range(8):
            x, y, z, w = _words(tile, b * 512 + lane * 16)
            _place32(Q, g, t, b * 32, (x, z, y, w))
    return Q


def test_operand_position_is_a_permutation_matching_the_b_fragment():
    # lane t's 8-byte word of a 32-span holds inputs 4t..4t+3 then 16+4t..16+4t+3
    pos = [((k & 15) >> 2) * 8 + ((k >> 4) & 1) * 4 + (k & 3) for k in range(32)]
    assert sorted(pos) == list(range(32))
    for t in range(4):
        assert [pos.index(8 * t + i) for i in range(8)] == [4 * t, 4 * t + 1, 4 * t + 2, 4 * t + 3,
                                                          16 + 4 * t, 17 + 4 * t, 18 + 4 * t, 19 + 4 * t]


def raw_integers(kind, raw, rows, cols):
    elems, size = H.BLOCK[kind]
    blocks = raw.reshape(rows, cols // elems, size)
    if kind == H.Q4_K:
        qs = blocks[:, :, 16:].reshape(rows, -1, 4, 32)
        q = np.empty((rows, cols // 256, 8, 32), dtype=np.int64)
        q[:, :, 0::2] = qs & 0x0F
        q[:, :, 1::2] = qs >> 4
        return q.reshape(rows, cols)
    if kind == H.Q6_K:
        ql = blocks[:, :, :128].reshape(rows, -1, 2, 2, 32)
        qh = blocks[:, :, 128:192].reshape(rows, -1, 2, 32)
        q = np.empty((rows, cols // 256, 2, 4, 32), dtype=np.int64)
        for v in range(4):
            q[:, :, :, v] = ((ql[:, :, :, v & 1] >> (0 if v < 2 else 4)) & 0x0F) | (((qh >> (2 * v)) & 3) << 4)
        return q.reshape(rows, cols)
    return (blocks[:, :, 2:].view(np.int8).astype(np.int64) + 128).reshape(rows, cols)


@pytest.mark.parametrize("kind,tile_bytes,emulate", [(H.Q4_K, 2304, emulate_q4k), (H.Q6_K, 3360, emulate_q6k),
                                                     (H.Q8_0, 4352, emulate_q8_0)])
def test_repack_feeds_the_mma_fragment_the_raw_integers(built_library, kind, tile_bytes, emulate):
    from ribn_b200 import ops
    rng = np.random.default_rng(kind)
    rows, cols = 40, 512  # 3 row tiles (last one ragged), 2 k tiles
    elems, size = H.BLOCK[kind]
    raw = rng.integers(0, 256, size=rows * (cols // elems) * size, dtype=np.uint8)
    packed = ops.repack(kind, raw, rows, cols)
    assert packed.size == 3 * 2 * tile_bytes
    want = raw_integers(kind, raw, rows, cols)
    blocks = raw.reshape(rows, cols // elems, size)
    for rt in range(3):
        for kb in range(2):
            tile = packed[(rt * 2 + kb) * tile_bytes:(rt * 2 + kb + 1) * tile_bytes]
            got = emulate(tile)
            live = min(16, rows - rt * 16)
            assert np.array_equal(got[:live], want[rt * 16:rt * 16 + live, kb * 256:(kb + 1) * 256])
            if kind == H.Q8_0:
                assert np.all(got[live:] == 128)          # padding rows decode to q = 0
            else:
                assert np.all(got[live:] == 0)
            for r in range(live):
                row = rt * 16 + r
                if kind == H.Q4_K:
                    assert np.array_equal(tile[2048 + r * 16:2048 + r * 16 + 16], blocks[row, kb, :16])
                elif kind == H.Q6_K:
                    assert np.array_equal(tile[3072 + r * 16:3072 + r * 16 + 16], blocks[row, kb, 192:208])
                    assert np.array_equal(tile[3328 + r * 2:3328 + r * 2 + 2], blocks[row, kb, 208:210])
                else:
                    for b in range(8):
                        assert np.array_equal(tile[4096 + r * 16 + b * 2:4096 + r * 16 + b * 2 + 2],
                                              blocks[row, kb * 8 + b, 0:2])


def test_compute_entry_points_fail_loudly_without_a_gpu(built_library):
    """On a machine without a CUDA device every compute call reports an error
    instead of computing on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import ribn_b200
    with pytest.raises(ribn_b200.ExecutionError, match="no CUDA device"):
        ribn_b200.QwenB200(H.TINY)
    with pytest.raises(RuntimeError, match="no usable CUDA device"):
        ribn_b200.ops.rms_norm(np.ones(4, np.float32), np.ones(4, np.float32), 1e-6)


def test_create_rejects_a_context_beyond_the_attention_span_limit(built_library):
    """context_tokens above 1024 spans x 64 keys is refused when the executor is created (before any
    device is touched), not at the first step that would exceed the attention launcher's limit."""
    import ribn_b200
    with pytest.raises(ribn_b200.ExecutionError, match="65536"):
        ribn_b200.QwenB200(H.TINY, context_tokens=65537, max_sequences=1, max_batch_tokens=16)
