"""The allocation-free attention entry point against the ordinary one.

Some callers of this library must not allocate device memory at call time: code that runs while
a CUDA stream is being captured into a graph, and serving loops whose device memory is handed
out once at start-up.  `ribn_b200_attention_noalloc` serves them by keeping its span scratch in
an array built into the library.  This test feeds both entry points the same paged K/V and
queries and checks that the results agree, twice in a row (the second call finds the previous
call's contents in the shared scratch).  The file name sorts last on purpose: a run that stops
at the first failure has then already run every other test."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOLERANCE = 1e-3  # the attention tolerance used throughout the GPU tests


def _case(rng, rows, tokens, q_heads, kv_heads, head_dim):
    pages = (tokens + 15) // 16
    table = rng.permutation(pages).astype(np.int32)
    q = rng.normal(0, 1, size=(rows, q_heads * head_dim)).astype(np.float32)
    k = rng.normal(0, 1, size=(pages * 16, kv_heads * head_dim)).astype(np.float16).view(np.uint16)
    v = rng.normal(0, 1, size=(pages * 16, kv_heads * head_dim)).astype(np.float16).view(np.uint16)
    return q, k, v, table


def test_noalloc_attention_matches_allocating_entry_point_twice(built_library):
    import torch
    from ribn_b200 import lib, ops
    rng = np.random.default_rng(77)
    dev = torch.device("cuda", 0)
    for call, (rows, tokens, qh, kvh, hd, window) in enumerate([(3, 700, 32, 8, 128, 0), (2, 1000, 16, 8, 128, 200)]):
        q, k, v, table = _case(rng, rows, tokens, qh, kvh, hd)
        want = ops.attention(q, k, v, table, tokens, rows, qh, kvh, hd, window=window)
        d_q = torch.from_numpy(q).to(dev)
        d_k = torch.from_numpy(k.view(np.int16)).to(dev)
        d_v = torch.from_numpy(v.view(np.int16)).to(dev)
        d_table = torch.from_numpy(table).to(dev)
        d_pos = torch.arange(tokens - rows, tokens, dtype=torch.int32, device=dev)
        d_out = torch.empty((rows, qh * hd), dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        err = C.create_string_buffer(512)
        stream = torch.cuda.current_stream(dev).cuda_stream
        before = torch.cuda.current_device()
        rc = lib().ribn_b200_attention_noalloc(0, C.c_void_p(stream), C.c_void_p(d_q.data_ptr()),
                                               C.c_void_p(d_k.data_ptr()), C.c_void_p(d_v.data_ptr()),
                                               C.c_void_p(d_table.data_ptr()), C.c_void_p(d_pos.data_ptr()), rows,
                                               tokens, qh, kvh, hd, window, C.c_void_p(d_out.data_ptr()), err, len(err))
        assert rc == 0, err.value.decode()
        assert torch.cuda.current_device() == before   # the caller's current device is left as it was
        torch.cuda.synchronize()
        got = d_out.cpu().numpy()
        assert np.max(np.abs(got - want)) < TOLERANCE, (call, float(np.max(np.abs(got - want))))
        if window == 0:
            # ... and directly against the CPU oracle, for the last row (it sees every key)
            from oracle import binding as orc
            order = table[np.arange(tokens) // 16] * 16 + np.arange(tokens) % 16
            ref = orc.attention(q[rows - 1], k[order].reshape(-1), v[order].reshape(-1), tokens, qh, kvh, hd)
            assert np.max(np.abs(got[rows - 1] - ref)) < TOLERANCE


def test_noalloc_attention_refuses_sizes_beyond_its_scratch(built_library):
    import torch
    from ribn_b200 import lib
    dev = torch.device("cuda", 0)
    dummy = torch.zeros(16, dtype=torch.float32, device=dev)
    err = C.create_string_buffer(512)
    p = C.c_void_p(dummy.data_ptr())
    # 64 rows x 32 heads x 128 spans x 130 floats = 34 M floats > 2 M
    rc = lib().ribn_b200_attention_noalloc(0, None, p, p, p, p, p, 64, 8192, 32, 8, 128, 0, p, err, len(err))
    assert rc != 0 and b"exceeds the built-in scratch" in err.value
    rc = lib().ribn_b200_attention_noalloc(0, None, p, p, p, p, p, 1, 64, 6, 2, 32, 0, p, err, len(err))
    assert rc != 0 and b"head_dim" in err.value
