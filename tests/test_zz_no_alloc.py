"""The attention entry point that allocates nothing, called through its
exported C symbol, against the ordinary entry point.

Some callers of the kernel library cannot hand it scratch memory: they gave
all device memory to an arena of their own, or they run where cudaMalloc is
forbidden.  For them ``yalm_attention_no_alloc`` keeps the split-KV scratch in
a fixed 8 MiB array inside the library.  This test makes two calls in a row
(the array keeps the first call's contents) and checks both against
``yalm_attention``, and checks that a request beyond the array is refused.
The file sorts last so that a run that stops at the first failure has already
run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _args(q, kv_step, kc, vc, token_seq, q_start, seq_slot, slot_pos, out):
    return [ctypes.c_void_p(t.data_ptr()) for t in
            (q, kv_step, kc, vc, token_seq, q_start, seq_slot, slot_pos, out)]


def _case(dt, H, G, hd, cap, window, lens, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    B = len(lens)
    n_slots = B + 2
    slots = list(range(1, B + 1))
    kc = torch.randn(n_slots, G, cap, hd, device=DEV, generator=g).to(dt)
    vc = torch.randn(n_slots, G, cap, hd, device=DEV, generator=g).to(dt)
    q = torch.randn(B, H * hd, device=DEV, generator=g).to(dt)
    kv_step = torch.randn(B, 2, G, hd, device=DEV, generator=g).to(dt)
    slot_pos = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
    slot_pos[torch.tensor(slots, device=DEV)] = torch.tensor(lens, dtype=torch.int32, device=DEV)
    ar = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
    return q, kv_step, kc, vc, ar[:B].contiguous(), ar, seq_slot, slot_pos


def test_no_alloc_attention_matches_the_ordinary_entry_point_twice():
    from yalm_b200.csrc import ops
    lib = ops.lib()
    fn = lib.yalm_attention_no_alloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 9 + [ctypes.c_int] * 8 + [ctypes.c_void_p]
    cap_fn = lib.yalm_attention_no_alloc_capacity
    cap_fn.restype = ctypes.c_longlong
    capacity_floats = cap_fn()
    assert capacity_floats == 2 * 1024 * 1024
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    class Batch:
        pass

    # two different calls in a row: the second finds the first one's leftovers in the array
    for dt, H, G, hd, cap, window, lens, nsplit, tol in [
            (torch.bfloat16, 8, 2, 64, 512, None, [500, 3, 77, 260], 7, 1.6e-2),
            (torch.float32, 6, 3, 48, 96, 40, [90, 41, 12], 3, 3e-6)]:
        q, kv_step, kc, vc, token_seq, q_start, seq_slot, slot_pos = _case(
            dt, H, G, hd, cap, window, lens, seed=hd)
        B = len(lens)
        assert B * H * nsplit * (hd + 2) <= capacity_floats
        out = torch.zeros(B, H * hd, device=DEV, dtype=dt)
        rc = fn(*_args(q, kv_step, kc, vc, token_seq, q_start, seq_slot, slot_pos, out),
                ops.dtype_code(dt), B, H, G, hd, cap, int(window or 0), nsplit, stream)
        assert rc == 0, rc
        b = Batch()
        b.token_seq, b.q_start, b.seq_slot = token_seq, q_start, seq_slot
        ref = torch.zeros_like(out)
        part_o = torch.empty(B * H * nsplit * hd, device=DEV)
        part_ml = torch.empty(B * H * nsplit * 2, device=DEV)
        ops.attention(q, kv_step, kc, vc, b, slot_pos, ref, H, G, hd, cap, window, nsplit,
                      part_o, part_ml)
        torch.cuda.synchronize()
        assert (out.float() - ref.float()).abs().max().item() <= tol
        assert ref.float().abs().max().item() > 0.01

    # beyond the array: refused, nothing launched, the output untouched
    q, kv_step, kc, vc, token_seq, q_start, seq_slot, slot_pos = _case(
        torch.bfloat16, 32, 8, 128, 64, None, [60] * 64, seed=1)
    out = torch.full((64, 32 * 128), 3.0, device=DEV, dtype=torch.bfloat16)
    nsplit = 16
    assert 64 * 32 * nsplit * (128 + 2) > capacity_floats
    rc = fn(*_args(q, kv_step, kc, vc, token_seq, q_start, seq_slot, slot_pos, out),
            ops.BF16, 64, 32, 8, 128, 64, 0, nsplit, stream)
    torch.cuda.synchronize()
    assert rc == -7
    assert torch.all(out == 3.0)
