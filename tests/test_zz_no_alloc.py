"""The allocation-free entry point, `patina_gemm_bf16_tn_skinny_noalloc`.

Who needs it: callers that are not allowed to allocate device memory when they call a GEMM --
code inside an allocator's own callback, a server whose device memory was carved up and audited
at start-up, a loop that cannot take cudaMalloc's device-wide synchronisation. The regular
entry points keep growable scratch in a context; this one keeps its scratch in a fixed array
inside the library and refuses problems that do not fit.

Checked here, through the C ABI: its output equals the regular stream-K entry point's (same
kernel, same partition, so bit for bit, which is inside the suite's tolerance) on two calls in
a row with different operands -- the second call meets the first one's leftovers in the shared
scratch; device memory in use does not change across the calls after the first (the first
call on a device is the documented warm-up: with lazy loading it is when the driver brings in
the module and the array); and oversize or out-of-range problems are refused with a message.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def call_noalloc(lib, A, B, out, alpha=1.0):
    err = C.create_string_buffer(512)
    M, K = A.shape
    N = B.shape[0]
    rc = lib.patina_gemm_bf16_tn_skinny_noalloc(
        A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), out.data_ptr(), out.stride(0),
        M, N, K, float(alpha), torch.cuda.current_stream().cuda_stream, err, len(err))
    return rc, err.value.decode()


def test_noalloc_matches_regular_entry_point_twice_in_a_row(oracle_mod):
    import numpy as np
    import patina_b200
    from patina_b200 import GemmConfig, inputs, lib as L
    lib = L.load()
    ctx = patina_b200.GemmContext(0)
    # Shapes whose weight tiles are split across CTAs, so the scratch array is really used:
    # 28 tiles x 64 k-blocks and 23 tiles x 33 k-blocks over 148 CTAs.
    for call, (M, N, K, alpha) in enumerate([(48, 3584, 4096, 1.0), (16, 2900, 2112, 0.5)]):
        A, B = inputs.make_operands("llm", M, N, K, seed=100 + call)
        dA, dB = A.cuda(), B.cuda()
        ldc = (N + 7) // 8 * 8
        want = torch.empty((M, ldc), dtype=torch.bfloat16, device="cuda")[:, :N]
        ctx.gemm_tn(dA, dB, out=want, alpha=alpha, config=GemmConfig(0, 0, 0, 0, 0, 0, 1))
        ctx.status()
        got = torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device="cuda")[:, :N]
        if call == 0:
            rc, msg = call_noalloc(lib, dA, dB, got, alpha)      # the warm-up call for this device
            assert rc == L.OK, msg
            got.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc, msg = call_noalloc(lib, dA, dB, got, alpha)
        assert rc == L.OK, msg
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "device memory in use changed across the call"
        assert torch.equal(got, want), f"call {call}: differs from the regular entry point"
        # and both are right: the suite's tolerance against the oracle
        wa = oracle_mod.bf16_bits_to_f32(A.view(torch.int16).numpy().view(np.uint16))
        wb = oracle_mod.bf16_bits_to_f32(B.view(torch.int16).numpy().view(np.uint16))
        ref = oracle_mod.scale_round_bf16(oracle_mod.ref_gemm_tn(wa, wb), alpha)
        ok, me, mx, fr = oracle_mod.compare_norm(got.float().cpu().numpy(), ref, 1e-2, 1e-3)
        assert ok, f"call {call}: max|d|={me:.4g} max|ref|={mx:.4g} fro_rel={fr:.4g}"
    ctx.close()


def test_noalloc_refuses_what_does_not_fit():
    from patina_b200 import lib as L
    lib = L.load()
    big_a = torch.zeros((128, 8192), dtype=torch.bfloat16, device="cuda")
    big_b = torch.zeros((28672, 8192), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((128, 28672), dtype=torch.bfloat16, device="cuda")
    rc, msg = call_noalloc(lib, big_a, big_b, out)   # needs 29 MB of partial tiles; 16 MiB are there
    assert rc == L.ERR_INVALID_ARG and "scratch" in msg and "29360128" in msg
    a = torch.zeros((130, 64), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((256, 64), dtype=torch.bfloat16, device="cuda")
    rc, msg = call_noalloc(lib, a, b, torch.zeros((130, 256), dtype=torch.bfloat16, device="cuda"))
    assert rc == L.ERR_INVALID_ARG and "1..128" in msg
    rc, msg = call_noalloc(lib, a[:16, :60], b[:, :60], out[:16, :256])   # K = 60 with lda = 64 is legal ...
    assert rc == L.OK, msg
    odd = torch.zeros((16, 60), dtype=torch.bfloat16, device="cuda")       # ... a 120-byte row pitch is not
    rc, msg = call_noalloc(lib, odd, b[:, :60], out[:16, :256])
    assert rc == L.ERR_INVALID_ARG and "16 bytes" in msg
    torch.cuda.synchronize()
