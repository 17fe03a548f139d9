"""Each kernel alone against a plain 32-bit reference of the same operation, at
sizes other than the engine's tiny configurations, with inputs built so that a
fault shows: a far key among hundreds, a window's edge, a wrapped ring, a slot."""
import math

import pytest
import torch

from plain_model import plain_argmax, plain_attention, plain_inv_freq, plain_rmsnorm, plain_rope

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# the 16-bit types with one rounding step of each (2^-8 for bfloat16's 8 bits of
# mantissa, 2^-11 for float16's 11)
HALF = [(torch.bfloat16, 2 ** -8), (torch.float16, 2 ** -11)]


@pytest.fixture(scope="module")
def ops():
    from yalm_b200.csrc import ops as o
    o.lib()
    return o


class B:
    """The index arrays of a ragged batch."""

    def __init__(self, q_lens, slots):
        qs = [0]
        for q in q_lens:
            qs.append(qs[-1] + q)
        self.n_seqs, self.n_tokens, self.q_lens, self.slots = len(q_lens), qs[-1], q_lens, slots
        self.q_start = torch.tensor(qs, dtype=torch.int32, device=DEV)
        self.seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
        self.token_seq = torch.tensor(sum([[i] * q for i, q in enumerate(q_lens)], []),
                                      dtype=torch.int32, device=DEV)


def test_embedding_gathers_rows_and_flags_bad_ids(ops):
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        table = torch.randn(1000, 200, device=DEV).to(dt)
        tok = torch.randint(0, 1000, (77,), device=DEV, dtype=torch.int32)
        x = torch.empty(77, 200, device=DEV)
        ops.embed(tok, table, x, status)
        assert torch.equal(x, table.float()[tok.long()]) and status.item() == 0
    tok[3] = 1000
    ops.embed(tok, table, x, status)
    assert status.item() == ops.ERR_TOKEN_RANGE


@pytest.mark.parametrize("dim", [40, 200, 1000, 4096, 5000])
def test_rmsnorm_with_partials_and_gather(ops, dim):
    x = torch.randn(23, dim, device=DEV) * 3
    w = torch.randn(dim, device=DEV)
    parts = torch.randn(4, 23, dim, device=DEV)
    ref = plain_rmsnorm(x.cpu(), w.cpu(), 1e-6)
    out = torch.empty(23, dim, device=DEV)
    xc = x.clone()
    ops.rmsnorm(xc, w, out, 1e-6)
    assert torch.equal(xc, x)
    assert (out.cpu() - ref).abs().max() <= 2e-6 * ref.abs().max()
    xs = x + parts.sum(0)
    ref = plain_rmsnorm(xs.cpu(), w.cpu(), 1e-6)
    ops.rmsnorm(xc, w, out, 1e-6, partials=parts, n_partials=4)
    assert (out.cpu() - ref).abs().max() <= 4e-6 * ref.abs().max()
    assert (xc - xs).abs().max() <= 1e-5                        # the residual sum was written back
    rows = torch.tensor([22, 0, 7, 7], dtype=torch.int32, device=DEV)
    for dt, eps in HALF:
        outg = torch.empty(4, dim, device=DEV, dtype=dt)
        xc = x.clone()
        ops.rmsnorm(xc, w, outg, 1e-6, partials=parts, n_partials=4, rows=rows)
        assert torch.equal(xc, x)                               # a gather leaves x alone
        assert (outg.float().cpu() - ref[rows.long().cpu()]).abs().max() <= 2 * eps * ref.abs().max()


def _paired_silu(ref):
    """silu(gate)*up when the columns of ref come as 16 gate columns followed by the 16
    up columns of the same features (the last group may be cut short by the caller)."""
    M, N = ref.shape
    r = ref.reshape(M, N // 32, 2, 16)
    g, u = r[:, :, 0], r[:, :, 1]
    return (g / (1 + torch.exp(-g)) * u).reshape(M, N // 2)


def test_silu_mul_sums_partials(ops):
    gu = torch.randn(3, 11, 2 * 333, device=DEV) * 2
    out = torch.empty(11, 333, device=DEV)
    ops.silu_mul(gu, out, n_partials=3)
    s = gu.sum(0).cpu()
    g, u = s[:, :333], s[:, 333:]
    ref = g / (1 + torch.exp(-g)) * u
    assert (out.cpu() - ref).abs().max() <= 1e-5 * ref.abs().max()
    gu = torch.randn(2, 7, 2 * 336, device=DEV) * 2            # paired columns
    ref = _paired_silu(gu.sum(0).cpu())
    for dt, eps in HALF:
        out = torch.empty(7, 336, device=DEV, dtype=dt)
        ops.silu_mul(gu, out, n_partials=2, paired=True)
        assert (out.float().cpu() - ref).abs().max() <= eps * ref.abs().max()


@pytest.mark.parametrize("shape", [(1, 70, 50), (65, 129, 17), (300, 520, 260)])
def test_fma_matrix_product_is_true_32_bit(ops, shape):
    M, N, K = shape
    a, w = torch.randn(M, K, device=DEV), torch.randn(N, K, device=DEV)
    ref = (a.double() @ w.double().T)
    out = torch.empty(M, N, device=DEV)
    ops.gemm_simt(a, w, out)
    # 32-bit accumulation: error ~ sqrt(K) * 2^-24 * |a||w|; a 10-bit mantissa mode would give 1e-3
    assert (out.double() - ref).abs().max() <= 3e-6 * math.sqrt(K) * ref.abs().max()
    ops.gemm_simt(a, w, out, accumulate=True)
    assert (out.double() - 2 * ref).abs().max() <= 6e-6 * math.sqrt(K) * ref.abs().max()
    # a row's result does not depend on the other rows of the batch
    one = torch.empty(1, N, device=DEV)
    ops.gemm_simt(a[M // 2:M // 2 + 1].contiguous(), w, one)
    ops.gemm_simt(a, w, out)
    assert torch.equal(one[0], out[M // 2])
    # mixed storage: bfloat16 activations on a matrix kept in 32 bits
    ah = a.to(torch.bfloat16)
    ops.gemm_simt(ah, w, out)
    assert (out.double() - ah.double() @ w.double().T).abs().max() <= 3e-6 * math.sqrt(K) * ref.abs().max()


@pytest.mark.parametrize("shape", [(1, 128, 64), (3, 200, 72), (16, 384, 512), (40, 1000, 320),
                                   (64, 2048, 1024), (130, 300, 88), (256, 512, 256), (700, 640, 448)])
@pytest.mark.parametrize("dt, eps", HALF)
def test_tcgen05_matrix_product_all_epilogues(ops, shape, dt, eps):
    M, N, K = shape
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    a = (torch.randn(M, K, device=DEV) * 0.5).to(dt)
    w = (torch.randn(N, K, device=DEV) * 0.5).to(dt)
    ref = a.double() @ w.double().T
    tol = 2e-6 * math.sqrt(K) * ref.abs().max()
    out = torch.full((M, N), 7.0, device=DEV)
    ops.gemm_tc(a, w, out, ops.GEMM_STORE, status)
    assert (out.double() - ref).abs().max() <= tol
    ops.gemm_tc(a, w, out, ops.GEMM_ADD, status)
    assert (out.double() - 2 * ref).abs().max() <= 2 * tol
    outh = torch.zeros(M, N, device=DEV, dtype=dt)
    ops.gemm_tc(a, w, outh, ops.GEMM_STORE, status)
    assert (outh.double() - ref).abs().max() <= eps * ref.abs().max()
    nkb = -(-K // 64)
    for S in sorted({1, min(2, nkb), min(5, nkb)}):
        per = -(-nkb // S)
        if (S - 1) * per >= nkb:
            continue
        part = torch.full((S, M, N), 3.0, device=DEV)
        ops.gemm_tc(a, w, part, ops.GEMM_SPLIT, status, splits=S)
        assert (part.sum(0).double() - ref).abs().max() <= tol, S
    g, u = ref[:, :N // 2], ref[:, N // 2:]
    r2 = g / (1 + torch.exp(-g)) * u
    o2 = torch.zeros(M, N // 2, device=DEV)
    ops.gemm_tc(a, w, o2, ops.GEMM_SILU_MUL, status)
    assert (o2.double() - r2).abs().max() <= 4e-6 * math.sqrt(K) * max(1.0, r2.abs().max())
    if N % 32 == 0:
        r4 = _paired_silu(ref)
        o4 = torch.full((M, N // 2), 9.0, device=DEV)
        ops.gemm_tc(a, w, o4, ops.GEMM_SILU_PAIRED, status)
        assert (o4.double() - r4).abs().max() <= 4e-6 * math.sqrt(K) * max(1.0, r4.abs().max())
    assert status.item() == 0


def test_tcgen05_refuses_what_tma_cannot_address(ops):
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    a = torch.zeros(4, 36, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(128, 36, device=DEV, dtype=torch.bfloat16)
    assert not ops.gemm_tc_usable(a, w)
    with pytest.raises(ops.KernelError, match="refused"):
        ops.gemm_tc(a, w, torch.zeros(4, 128, device=DEV), ops.GEMM_STORE, status)
    with pytest.raises(ops.KernelError, match="split"):
        ops.gemm_tc(torch.zeros(4, 64, device=DEV, dtype=torch.bfloat16),
                    torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16),
                    torch.zeros(2, 4, 128, device=DEV), ops.GEMM_SPLIT, status, splits=2)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
def test_rotary_kernel_for_prompts_agrees_with_the_general_one(ops, dt):
    """With 512 tokens or more in one slice the rotary kernel takes four tokens per block.
    The same input as two slices (the second one zero) goes through the general kernel:
    rotated queries, step keys and values and the ring rows must agree to the bit.  The
    prompts lie on top of earlier positions and one of them overruns its ring."""
    H, G, hd, cap = 6, 2, 64, 100
    lens, slots, past = [300, 7, 420], [2, 0, 1], [5, 0, 50]
    inv = plain_inv_freq(hd, 10000.0, None).to(DEV)
    b = B(lens, slots)
    N = b.n_tokens
    g = torch.Generator(device=DEV).manual_seed(4)
    qkv = torch.randn(N, (H + 2 * G) * hd, device=DEV, generator=g)
    two = torch.stack([qkv, torch.zeros_like(qkv)])
    got = []
    for src, n in ((qkv, 1), (two, 2)):
        slot_pos = torch.zeros(3, dtype=torch.int32, device=DEV)
        for s_, p_ in zip(slots, past):
            slot_pos[s_] = p_
        kc = torch.full((3, G, cap, hd), 7.0, device=DEV, dtype=dt)
        vc = torch.full((3, G, cap, hd), 7.0, device=DEV, dtype=dt)
        q_out = torch.empty(N, H * hd, device=DEV, dtype=dt)
        kv_step = torch.empty(N, 2, G, hd, device=DEV, dtype=dt)
        ops.rope_store(src, n, inv, b, q_out, kv_step, kc, vc, slot_pos, H, G, hd, cap)
        got.append((q_out, kv_step, kc, vc))
    for a_, b_ in zip(*got):
        assert torch.equal(a_, b_)
    # and against the plain rotation: the last token of the longest prompt
    t = N - 1
    pos = torch.tensor([past[2] + lens[2] - 1])
    ref = plain_rope(qkv[t].cpu().view(1, H + 2 * G, hd)[:, :H], pos, inv.cpu())
    assert (got[0][0][t].float().cpu().view(H, hd) - ref[0]).abs().max() <= (3e-6 if dt == torch.float32 else 3e-2)


def _rope_attend(ops, dt, H, G, hd, cap, window, q_lens, slots, n_slots, steps, nsplit_decode):
    """Drives rope_store + attention over several steps and returns the largest
    error against plain_rope + plain_attention on the whole sequences."""
    inv = plain_inv_freq(hd, 10000.0, None).to(DEV)
    slot_pos = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
    kc = torch.zeros(n_slots, G, cap, hd, device=DEV, dtype=dt)
    vc = torch.zeros_like(kc)
    hist = {s: [] for s in slots}
    worst = 0.0
    for step in range(steps):
        lens = q_lens if step == 0 else [1] * len(slots)
        b = B(lens, slots)
        N = b.n_tokens
        qkv = torch.randn(N, (H + 2 * G) * hd, device=DEV)
        q_out = torch.empty(N, H * hd, device=DEV, dtype=dt)
        kv_step = torch.empty(N, 2, G, hd, device=DEV, dtype=dt)
        ops.rope_store(qkv, 1, inv, b, q_out, kv_step, kc, vc, slot_pos, H, G, hd, cap)
        out = torch.empty(N, H * hd, device=DEV, dtype=dt)
        ns = 1 if step == 0 else nsplit_decode
        po = torch.empty(N * H * ns * hd, device=DEV)
        pml = torch.empty(N * H * ns * 2, device=DEV)
        ops.attention(q_out, kv_step, kc, vc, b, slot_pos, out, H, G, hd, cap, window, ns, po, pml)
        qs = b.q_start.tolist()
        for i, s in enumerate(slots):
            hist[s].append(qkv[qs[i]:qs[i + 1]].cpu().view(-1, H + 2 * G, hd))
            allt = torch.cat(hist[s])
            T = allt.shape[0]
            pos = torch.arange(T)
            q = plain_rope(allt[:, :H], pos, inv.cpu()).to(dt).float()
            k = plain_rope(allt[:, H:H + G], pos, inv.cpu()).to(dt).float()
            v = allt[:, H + G:].to(dt).float()
            ref = plain_attention(q, k, v, window)[T - lens[i]:]
            got = out[qs[i]:qs[i + 1]].float().cpu().view(-1, H, hd)
            worst = max(worst, float((got - ref).abs().max()))
        ops.advance(b, slot_pos)
    return worst


@pytest.mark.parametrize("dt, tol", [(torch.float32, 3e-6), (torch.bfloat16, 1.6e-2), (torch.float16, 2e-3)])
@pytest.mark.parametrize("H, G, hd, cap, window", [
    (8, 8, 16, 96, None),      # no grouping
    (10, 2, 80, 96, None),     # 5 query heads per kv head, head size 80
    (16, 1, 64, 24, 24),       # one kv head, a ring of 24 rows shorter than the prompt
    (4, 4, 256, 96, 50),       # the largest head, window inside a larger ring
    (6, 3, 112, 40, 40),
])
def test_rotary_cache_write_and_attention(ops, dt, tol, H, G, hd, cap, window):
    err = _rope_attend(ops, dt, H, G, hd, cap, window, q_lens=[33, 1, 60], slots=[4, 0, 2],
                       n_slots=5, steps=10, nsplit_decode=3)
    assert err <= tol, err


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
def test_attention_finds_a_far_key_a_window_edge_and_a_wrapped_row(ops, dt):
    """Keys are one-hot, queries 1e3 times a one-hot: the output is the value
    of exactly one position.  Position 3 among 700; the oldest key inside a
    window; the key just outside it; a ring row that has been overwritten."""
    H = G = 1
    hd = 64
    for window, cap, T, targets in [(None, 1024, 700, [3, 0, 699, 350]),
                                    (64, 64, 700, [699, 636, 650])]:
        n_slots = 3
        slot = 1
        kc = torch.zeros(n_slots, G, cap, hd, device=DEV, dtype=dt)
        vc = torch.zeros_like(kc)
        # keys: position p has key e_{p % 64} scaled by (1 + p/1000) so that equal directions differ
        pos = torch.arange(T)
        keys = torch.zeros(T, hd)
        keys[pos, pos % hd] = 1.0
        vals = torch.zeros(T, hd)
        vals[pos, (pos * 7) % hd] = 1.0 + pos.float() / 1024.0
        live = pos if window is None else pos[T - window:]
        kc[slot, 0, live % cap] = keys[live].to(dt).to(DEV)
        vc[slot, 0, live % cap] = vals[live].to(dt).to(DEV)
        slot_pos = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
        slot_pos[slot] = T - 1                       # the query is the token at position T-1
        b = B([1], [slot])
        kv_step = torch.zeros(1, 2, G, hd, device=DEV, dtype=dt)
        kv_step[0, 0, 0] = keys[T - 1].to(dt)
        kv_step[0, 1, 0] = vals[T - 1].to(dt)
        for tgt in targets:
            # a bias towards late positions that only the one-hot match can beat
            q = torch.zeros(1, hd, device=DEV)
            q[0, tgt % hd] = 1000.0
            lo = 0 if window is None else T - window
            cands = [p for p in range(lo, T) if p % hd == tgt % hd]
            for ns in (1, 4):
                out = torch.empty(1, hd, device=DEV, dtype=dt)
                po = torch.empty(ns * hd, device=DEV)
                pml = torch.empty(ns * 2, device=DEV)
                ops.attention(q.to(dt), kv_step, kc, vc, b, slot_pos, out, H, G, hd, cap, window,
                              ns, po, pml)
                ref = torch.stack([vals[p] for p in cands]).mean(0)
                assert (out[0].float().cpu() - ref.to(dt).float()).abs().max() < 2e-2, (window, tgt, ns)
        if window is not None:
            # the key just outside the window (position T-1-window) must not be seen
            outside = T - 1 - window
            assert outside % hd == (T - 1) % hd       # same direction as the newest key
            q = torch.zeros(1, hd, device=DEV)
            q[0, outside % hd] = 1000.0
            out = torch.empty(1, hd, device=DEV, dtype=dt)
            ops.attention(q.to(dt), kv_step, kc, vc, b, slot_pos, out, H, G, hd, cap, window, 1)
            assert abs(out[0, ((T - 1) * 7) % hd].item() - vals[T - 1].max().item()) < 2e-2


def test_sampling_greedy_and_temperature(ops):
    V = 5003
    logits = torch.randn(6, V, device=DEV) * 4
    logits[2, 17] = logits[2, 4000] = 60.0                      # a tie: the first index wins
    slot_pos = torch.tensor([5, 6, 7, 8, 9, 10], dtype=torch.int32, device=DEV)
    seq_slot = torch.arange(6, dtype=torch.int32, device=DEV)
    keys = torch.arange(6, dtype=torch.int32, device=DEV) + 100
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    ops.sample(logits, 0.0, 1, keys, seq_slot, slot_pos, out)
    assert out.tolist() == [plain_argmax(r) for r in logits.cpu()] and out[2].item() == 17
    for temp in (1.0, 0.3, 2.5):
        for seed in range(4):
            ops.sample(logits, temp, seed, keys, seq_slot, slot_pos, out)
            for r in range(6):
                u = ops.uniform01(seed, 100 + r, 5 + r)
                assert 0.0 <= u < 1.0
                c = torch.softmax(logits[r].double().cpu() / temp, 0).cumsum(0)
                t = out[r].item()
                lo = 0.0 if t == 0 else c[t - 1].item()
                assert lo - 1e-5 <= u <= c[t].item() + 1e-5, (temp, seed, r)
    # the draw depends on (seed, key, position) only, not on the row it sits in
    ops.sample(logits[3:4].contiguous(), 1.0, 2, keys[3:4].contiguous(), seq_slot[:1].contiguous(),
               slot_pos[3:4].contiguous(), out[:1])
    one = out[0].item()
    ops.sample(logits, 1.0, 2, keys, seq_slot, slot_pos, out)
    assert out[3].item() == one
    from yalm_b200 import sampling
    us = [sampling.uniform01(9, 1, i) for i in range(2000)]
    assert 0.45 < sum(us) / len(us) < 0.55 and len(set(us)) > 1990
    # seed and temperature read from device memory (what a captured step does) give the
    # same tokens as the same values passed as arguments
    for temp, seed in ((0.0, 5), (0.7, 2 ** 63 + 11), (1.9, 3)):
        ops.sample(logits, temp, seed, keys, seq_slot, slot_pos, out)
        want = out.tolist()
        params = torch.tensor(ops.sampling_params(temp, seed), dtype=torch.int64, device=DEV)
        ops.sample(logits, 123.0, 999, keys, seq_slot, slot_pos, out, params=params)
        assert out.tolist() == want, (temp, seed)


def test_a_bounded_wait_that_runs_out_is_reported_and_the_device_stays_usable(ops):
    """A kernel waits on a barrier that nobody arrives on, gives up after a millisecond
    and raises the status bit; the runtime turns it into an error and clears it."""
    from yalm_b200.parts import Runtime
    rt = Runtime(torch.float32, DEV)
    ops.wait_probe(1_000_000, rt.status)
    with pytest.raises(ops.KernelError, match="bounded barrier wait"):
        rt.check_status()
    rt.check_status()                                           # cleared
    with pytest.raises(ops.KernelError, match="refused"):
        ops.wait_probe(10 ** 10, rt.status)                     # limits beyond 100 ms are refused
    x = torch.arange(8, device=DEV).sum().item()                # the context still works
    assert x == 28


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
def test_ring_rows_written_from_the_step_buffer(ops, dt):
    """cache_write puts a step's keys and values where rope_store would have put them:
    only the positions the ring keeps, at row position % capacity, other rows untouched."""
    G, hd, cap, n_slots = 3, 24, 16, 4
    for hd in (24, 20):                                         # 16-byte rows and odd ones
        b = B([21, 1, 5], [2, 0, 3])
        slot_pos = torch.tensor([30, 0, 7, 13], dtype=torch.int32, device=DEV)
        kv = torch.randn(b.n_tokens, 2, G, hd, device=DEV).to(dt)
        kc = torch.full((n_slots, G, cap, hd), 7.0, device=DEV, dtype=dt)
        vc = torch.full_like(kc, 7.0)
        ops.cache_write(kv, b, kc, vc, slot_pos, G, hd, cap)
        want_k, want_v = torch.full_like(kc, 7.0), torch.full_like(vc, 7.0)
        qs = b.q_start.tolist()
        for i, slot in enumerate(b.slots):
            past, n = int(slot_pos[slot]), b.q_lens[i]
            for j in range(n):
                pos = past + j
                if pos >= past + n - cap:
                    want_k[slot, :, pos % cap] = kv[qs[i] + j, 0]
                    want_v[slot, :, pos % cap] = kv[qs[i] + j, 1]
        assert torch.equal(kc, want_k) and torch.equal(vc, want_v)


@pytest.mark.parametrize("dt, tol", [(torch.float32, 3e-6), (torch.bfloat16, 1.6e-2), (torch.float16, 2e-3)])
@pytest.mark.parametrize("H, G, hd, cap, window, chunk", [
    (8, 2, 128, 700, None, 64),     # chunks of 64 keys, the last one ragged
    (6, 3, 48, 40, 40, 32),         # a ring that wraps inside a chunk
    (5, 5, 16, 300, 100, 128),      # window inside a larger ring, one chunk
    (16, 2, 64, 512, None, 32),     # 8 query heads per kv head: two head groups
])
def test_decode_attention_from_staged_chunks(ops, dt, tol, H, G, hd, cap, window, chunk):
    """attention_decode (bulk copies into shared memory, chunks merged by the
    last block) against the plain attention over each sequence's visible keys,
    twice in a row (the counters must come back to zero)."""
    g = torch.Generator(device=DEV).manual_seed(hd + cap)
    lens = [1, 37, cap - 1, cap, 3 * cap + 5] if window else [1, 37, 200, cap - 1, cap]
    B, n_slots = len(lens), len(lens) + 3
    slots = [5, 0, 3, 7, 2][:B]
    kc = torch.randn(n_slots, G, cap, hd, device=DEV, generator=g).to(dt)
    vc = torch.randn(n_slots, G, cap, hd, device=DEV, generator=g).to(dt)
    q = torch.randn(B, H * hd, device=DEV, generator=g).to(dt)
    slot_pos = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
    for s, n in zip(slots, lens):
        slot_pos[s] = n - 1                                     # the query is the last position
    seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
    bound = max(lens)
    visible = min(bound, window) if window else bound
    mc = -(-visible // chunk)
    part_o = torch.empty(B * H * mc * hd, device=DEV)
    part_ml = torch.empty(B * H * mc * 2, device=DEV)
    counters = torch.zeros(B * G * -(-(H // G) // 4), dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for rep in range(2):
        out = torch.zeros(B, H * hd, device=DEV, dtype=dt)
        ops.attention_decode(q, kc, vc, seq_slot, slot_pos, out, part_o, part_ml, counters, status,
                             H, G, hd, cap, window, chunk, bound)
        torch.cuda.synchronize()
        assert status.item() == 0 and int(counters.abs().sum()) == 0
        for b, (s, n) in enumerate(zip(slots, lens)):
            lo = 0 if window is None else max(0, n - window)
            rows = torch.tensor([p % cap for p in range(lo, n)])
            k = kc[s][:, rows].permute(1, 0, 2).float().cpu()   # [keys, G, hd]
            v = vc[s][:, rows].permute(1, 0, 2).float().cpu()
            qq = torch.zeros(len(rows), H, hd)
            qq[-1] = q[b].float().cpu().view(H, hd)
            ref = plain_attention(qq, k, v, None)[-1]
            got = out[b].float().cpu().view(H, hd)
            assert (got - ref).abs().max().item() <= tol, (rep, b, n)
    # a bound that is too small is reported, not silently wrong
    ops.attention_decode(q, kc, vc, seq_slot, slot_pos, out, part_o, part_ml, counters, status,
                         H, G, hd, cap, window, chunk, 1)
    torch.cuda.synchronize()
    need = max(-(-(min(n, window) if window else n) // chunk) for n in lens)
    assert status.item() == (ops.ERR_CONTEXT_RANGE if need > 1 else 0)


@pytest.mark.parametrize("H, G, hd, cap, window", [
    (8, 2, 128, 256, None),
    (6, 3, 48, 40, 40),         # a ring shorter than the prompts
    (5, 5, 16, 300, 100),
    (16, 2, 64, 512, None),
    (4, 1, 112, 200, 70),
])
@pytest.mark.parametrize("dt, eps", HALF)
def test_tensor_core_prefill_attention(ops, H, G, hd, cap, window, dt, eps):
    """attention_prefill_mma against the plain attention: ragged prompts (one
    longer than 64-token tiles, one of a single token), then a second chunk of
    the same sequences on top of the cache (keys from the ring and from the step)."""
    inv = plain_inv_freq(hd, 10000.0, None).to(DEV)
    n_slots, slots = 4, [2, 0, 3]
    slot_pos = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
    kc = torch.zeros(n_slots, G, cap, hd, device=DEV, dtype=dt)
    vc = torch.zeros_like(kc)
    hist = {s: [] for s in slots}
    for lens in ([150, 1, 70], [20, 37, 1]):
        if window is None and max(a + b for a, b in zip([sum(x.shape[0] for x in hist[s]) for s in slots], lens)) > cap:
            continue
        b = B(lens, slots)
        N = b.n_tokens
        qkv = torch.randn(N, (H + 2 * G) * hd, device=DEV)
        q_out = torch.empty(N, H * hd, device=DEV, dtype=dt)
        kv_step = torch.empty(N, 2, G, hd, device=DEV, dtype=dt)
        # the ring is written after the attention: several tokens on top of a full
        # ring would otherwise replace keys that the first of them still sees
        ops.rope_store(qkv, 1, inv, b, q_out, kv_step, kc, vc, slot_pos, H, G, hd, cap,
                       write_cache=False)
        out = torch.empty(N, H * hd, device=DEV, dtype=dt)
        ops.attention_prefill_mma(q_out, kv_step, kc, vc, b, slot_pos, out, H, G, hd, cap, window)
        ref_simt = torch.empty_like(out)
        ops.attention(q_out, kv_step, kc, vc, b, slot_pos, ref_simt, H, G, hd, cap, window, 1)
        ops.rope_store(qkv, 1, inv, b, q_out, kv_step, kc, vc, slot_pos, H, G, hd, cap)
        qs = b.q_start.tolist()
        for i, s in enumerate(slots):
            hist[s].append(qkv[qs[i]:qs[i + 1]].cpu().view(-1, H + 2 * G, hd))
            allt = torch.cat(hist[s])
            T = allt.shape[0]
            pos = torch.arange(T)
            qq = plain_rope(allt[:, :H], pos, inv.cpu()).to(dt).float()
            kk = plain_rope(allt[:, H:H + G], pos, inv.cpu()).to(dt).float()
            vv = allt[:, H + G:].to(dt).float()
            ref = plain_attention(qq, kk, vv, window)[T - lens[i]:]
            got = out[qs[i]:qs[i + 1]].float().cpu().view(-1, H, hd)
            assert (got - ref).abs().max().item() <= 6.4 * eps, (lens, i)
        assert (out.float() - ref_simt.float()).abs().max().item() <= 6.4 * eps
        ops.advance(b, slot_pos)


@pytest.mark.parametrize("H, G, hd, cap, window", [
    (32, 8, 128, 700, None),
    (6, 3, 48, 40, 40),
    (40, 2, 64, 300, 100),      # 20 query heads per kv head: two head groups of the tile
    (3, 1, 32, 1000, None),
    (24, 2, 80, 200, None),     # 12 query heads per kv head: both 8-head tiles, one partly empty
    (4, 2, 64, 1700, None),     # 27 parts at one chunk per block
])
@pytest.mark.parametrize("warps", [4, 2])
@pytest.mark.parametrize("dt, eps", HALF)
def test_tensor_core_decode_attention(ops, H, G, hd, cap, window, dt, eps, warps):
    g = torch.Generator(device=DEV).manual_seed(hd + cap)
    lens = [1, 37, cap - 1, cap, 3 * cap + 5] if window else [1, 129, 200, cap - 1, cap]
    Bn, n_slots = len(lens), len(lens) + 3
    slots = [5, 0, 3, 7, 2]
    kc = torch.randn(n_slots, G, cap, hd, device=DEV, generator=g).to(dt)
    vc = torch.randn(n_slots, G, cap, hd, device=DEV, generator=g).to(dt)
    q = torch.randn(Bn, H * hd, device=DEV, generator=g).to(dt)
    slot_pos = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
    for s, n in zip(slots, lens):
        slot_pos[s] = n - 1
    seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
    bound = max(lens)
    counters = torch.zeros(Bn * G * -(-(H // G) // 16), dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for rep, cpc in enumerate((1, 3, 1000)):                   # merged parts ... one block per query
        mc = ops.decode_mma_parts(bound, window, cpc)
        part_o = torch.empty(Bn * H * mc * hd, device=DEV)
        part_ml = torch.empty(Bn * H * mc * 2, device=DEV)
        out = torch.zeros(Bn, H * hd, device=DEV, dtype=dt)
        ops.attention_decode_mma(q, kc, vc, seq_slot, slot_pos, out, part_o, part_ml, counters,
                                 status, H, G, hd, cap, window, bound, cpc, warps=warps)
        torch.cuda.synchronize()
        assert status.item() == 0 and int(counters.abs().sum()) == 0
        for b, (s, n) in enumerate(zip(slots, lens)):
            lo = 0 if window is None else max(0, n - window)
            rows = torch.tensor([p % cap for p in range(lo, n)])
            k = kc[s][:, rows].permute(1, 0, 2).float().cpu()
            v = vc[s][:, rows].permute(1, 0, 2).float().cpu()
            qq = torch.zeros(len(rows), H, hd)
            qq[-1] = q[b].float().cpu().view(H, hd)
            ref = plain_attention(qq, k, v, None)[-1]
            got = out[b].float().cpu().view(H, hd)
            assert (got - ref).abs().max().item() <= 6.4 * eps, (rep, b, n)


@pytest.mark.parametrize("paged", [False, True])
@pytest.mark.parametrize("H, G, hd, cap, window, S", [
    (32, 8, 128, 700, None, 6),
    (6, 3, 48, 40, 40, 1),
    (40, 2, 64, 300, 100, 3),     # 20 query heads per kv head: two head groups write the same new row
    (3, 1, 32, 1000, None, 9),
    (24, 2, 80, 200, None, 2),
])
@pytest.mark.parametrize("dt, eps", HALF)
def test_decode_attention_with_the_rotary_work_inside(ops, H, G, hd, cap, window, S, dt, eps, paged):
    """attention_decode_mma_fused against rope_store followed by attention_decode_mma, bit for
    bit: outputs and both caches.  Sequences whose new key opens a unit, ends one, lies in a
    unit that the block has staged before its wait or asks for later, and (windowed) lands on
    a ring row that holds an old key; few and many slices of the product; pages."""
    g = torch.Generator(device=DEV).manual_seed(hd + cap + S)
    lens = [1, 37, cap - 1, cap, 3 * cap + 5] if window else [1, 129, 200, cap - 1, cap, 33, 64, 65]
    Bn, n_slots = len(lens), len(lens) + 3
    slots = [5, 0, 3, 7, 2, 9, 1, 4][:Bn]
    inv = plain_inv_freq(hd, 10000.0, None).to(DEV)
    kc0 = torch.randn(n_slots, G, cap, hd, device=DEV, generator=g).to(dt)
    vc0 = torch.randn(n_slots, G, cap, hd, device=DEV, generator=g).to(dt)
    table = None
    if paged:
        kc0, vc0, table = _paged(kc0, vc0, seed=7)
    parts = torch.randn(S, Bn, (H + 2 * G) * hd, device=DEV, generator=g)
    slot_pos = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
    for s_, n in zip(slots, lens):
        slot_pos[s_] = n - 1                                    # the new token's position
    b = B([1] * Bn, slots)
    bound = max(lens)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    cs = torch.empty(Bn, hd // 2, 2, device=DEV)
    ops.rope_table(inv, b, slot_pos, cs)
    for cpc in (1, 3, 1000):
        mc = ops.decode_mma_parts(bound, window, cpc)
        res = []
        for fused in (False, True):
            kc, vc = kc0.clone(), vc0.clone()
            counters = torch.zeros(Bn * G * -(-(H // G) // 16), dtype=torch.int32, device=DEV)
            part_o = torch.empty(Bn * H * mc * hd, device=DEV)
            part_ml = torch.empty(Bn * H * mc * 2, device=DEV)
            out = torch.zeros(Bn, H * hd, device=DEV, dtype=dt)
            if fused:
                ops.attention_decode_mma_fused(parts, S, cs, kc, vc, b.seq_slot, slot_pos, out, part_o,
                                               part_ml, counters, status, H, G, hd, cap, window, bound,
                                               cpc, pages=table)
            else:
                q = torch.empty(Bn, H * hd, device=DEV, dtype=dt)
                kv_step = torch.empty(Bn, 2, G, hd, device=DEV, dtype=dt)
                ops.rope_store(parts, S, inv, b, q, kv_step, kc, vc, slot_pos, H, G, hd, cap, pages=table)
                ops.attention_decode_mma(q, kc, vc, b.seq_slot, slot_pos, out, part_o, part_ml, counters,
                                         status, H, G, hd, cap, window, bound, cpc, pages=table)
            torch.cuda.synchronize()
            assert status.item() == 0 and int(counters.abs().sum()) == 0
            res.append((out, kc, vc))
        for name, x, y in zip(("out", "k cache", "v cache"), res[0], res[1]):
            assert torch.equal(x, y), (name, cpc)


@pytest.mark.parametrize("shape", [(1, 128, 64), (130, 300, 88), (256, 256, 64), (300, 512, 128),
                                   (700, 640, 448), (1500, 1152, 320), (2048, 1024, 1024),
                                   (512, 9472, 64)])
@pytest.mark.parametrize("dt, eps", HALF)
def test_two_sm_matrix_product(ops, shape, dt, eps):
    """gemm_2sm: a cluster of two blocks per 256-feature tile (tcgen05.mma.cta_group::2),
    every epilogue, sizes that leave the second block of a pair partly or wholly empty.
    The token tile is 240 wherever its waves over the 74 pairs cost no more than those of
    256 (all shapes but the last: 37 feature tiles x 2 token tiles of 256 are one wave,
    x 3 of 240 would be two)."""
    M, N, K = shape
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    a = (torch.randn(M, K, device=DEV) * 0.5).to(dt)
    w = (torch.randn(N, K, device=DEV) * 0.5).to(dt)
    ref = a.double() @ w.double().T
    tol = 2e-6 * math.sqrt(K) * ref.abs().max()
    for rep in range(2):
        out = torch.full((M, N), 7.0, device=DEV)
        ops.gemm_2sm(a, w, out, ops.GEMM_STORE, status)
        assert (out.double() - ref).abs().max() <= tol
        ops.gemm_2sm(a, w, out, ops.GEMM_ADD, status)
        assert (out.double() - 2 * ref).abs().max() <= 2 * tol
        outh = torch.zeros(M, N, device=DEV, dtype=dt)
        ops.gemm_2sm(a, w, outh, ops.GEMM_STORE, status)
        assert (outh.double() - ref).abs().max() <= eps * ref.abs().max()
        g, u = ref[:, :N // 2], ref[:, N // 2:]
        r2 = g / (1 + torch.exp(-g)) * u
        o2 = torch.zeros(M, N // 2, device=DEV)
        ops.gemm_2sm(a, w, o2, ops.GEMM_SILU_MUL, status)
        assert (o2.double() - r2).abs().max() <= 4e-6 * math.sqrt(K) * max(1.0, r2.abs().max())
        if N % 32 == 0:
            r4 = _paired_silu(ref)
            o4 = torch.full((M, N // 2), 9.0, device=DEV, dtype=dt)
            ops.gemm_2sm(a, w, o4, ops.GEMM_SILU_PAIRED, status)
            assert (o4.double() - r4).abs().max() <= eps * max(1.0, r4.abs().max())
        # slices of K as 32-bit partial sums (what fills the idle pairs at a few hundred tokens)
        nkb = -(-K // 64)
        for S in (2, 3, 5):
            per = -(-nkb // S)
            if S > nkb or (S - 1) * per >= nkb:
                continue
            parts = torch.full((S, M, N), 7.0, device=DEV)
            ops.gemm_2sm(a, w, parts, ops.GEMM_SPLIT, status, splits=S)
            assert (parts.double().sum(0) - ref).abs().max() <= tol, S
            if S == 2:          # each slice is its own part of the sum
                first = a[:, :per * 64].double() @ w[:, :per * 64].double().T
                assert (parts[0].double() - first).abs().max() <= tol
        torch.cuda.synchronize()
        assert status.item() == 0


@pytest.mark.parametrize("H, G, hd, window", [(8, 2, 128, None), (4, 4, 64, None), (6, 3, 128, 100),
                                              (3, 1, 64, 37)])
@pytest.mark.parametrize("dt, eps", HALF)
def test_tcgen05_prefill_attention(ops, H, G, hd, window, dt, eps):
    """attention_prefill_tc (S and P.V in tensor memory) against the plain attention:
    ragged prompts from their first token: 300 tokens (a second block with one tile only),
    a single token, ends just past and at a tile, 700 tokens (three blocks of two tiles).
    On the second pass one early key of each prompt is made to dominate, and late ones
    grow, so the reference maximum of the rows is raised along the way."""
    inv = plain_inv_freq(hd, 10000.0, None).to(DEV)
    lens, slots, cap = [300, 1, 130, 128, 700], [2, 0, 3, 1, 4], 1024
    slot_pos = torch.zeros(5, dtype=torch.int32, device=DEV)
    kc = torch.zeros(5, G, cap, hd, device=DEV, dtype=dt)
    vc = torch.zeros_like(kc)
    b = B(lens, slots)
    N = b.n_tokens
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for rep in range(2):
        qkv = torch.randn(N, (H + 2 * G) * hd, device=DEV)
        if rep == 1:
            # keys grow with the position: later blocks keep raising the rows' maxima
            # (values halved: the output is then nearly one value row, and its own
            # rounding to bfloat16 must stay well inside the tolerance)
            ramp = 1.0 + torch.arange(N, device=DEV).float().remainder(701.0) / 100.0
            qkv.view(N, H + 2 * G, hd)[:, H:H + G] *= ramp[:, None, None]
            qkv.view(N, H + 2 * G, hd)[:, H + G:] *= 0.5
        q_out = torch.empty(N, H * hd, device=DEV, dtype=dt)
        kv_step = torch.empty(N, 2, G, hd, device=DEV, dtype=dt)
        ops.rope_store(qkv, 1, inv, b, q_out, kv_step, kc, vc, slot_pos, H, G, hd, cap)
        out = torch.full((N, H * hd), 9.0, device=DEV, dtype=dt)
        ops.attention_prefill_tc(q_out, kv_step, b, out, H, G, hd, window, status)
        torch.cuda.synchronize()
        assert status.item() == 0
        qs = b.q_start.tolist()
        for i in range(len(lens)):
            t = qkv[qs[i]:qs[i + 1]].cpu().view(-1, H + 2 * G, hd)
            pos = torch.arange(lens[i])
            qq = plain_rope(t[:, :H], pos, inv.cpu()).to(dt).float()
            kk = plain_rope(t[:, H:H + G], pos, inv.cpu()).to(dt).float()
            vv = t[:, H + G:].to(dt).float()
            ref = plain_attention(qq, kk, vv, window)
            got = out[qs[i]:qs[i + 1]].float().cpu().view(-1, H, hd)
            assert (got - ref).abs().max().item() <= 6.4 * eps, (rep, i)


@pytest.mark.parametrize("paged", [False, True])
@pytest.mark.parametrize("H, G, hd, cap, window", [(8, 2, 128, 1000, None), (4, 4, 64, 700, None),
                                                   (6, 3, 128, 960, 100), (3, 1, 64, 1024, 37)])
@pytest.mark.parametrize("dt, eps", HALF)
def test_tcgen05_prefill_attention_over_the_cache(ops, H, G, hd, cap, window, dt, eps, paged):
    """attention_prefill_tc_cache: prompts cut into three steps (the second and third read
    earlier keys from the cache: one block per sequence, or pages in a shuffled pool) against
    the plain attention over the whole sequences.  Lengths end inside a tile, at a tile, in a
    second block of two tiles; one sequence joins at the second step (its past is 0 there).
    The cache is filled with a large finite value first: a row beyond a sequence's end that
    reached a product would show."""
    inv = plain_inv_freq(hd, 10000.0, None).to(DEV)
    n_slots, slots = 5, [2, 0, 3, 4]
    slot_pos = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
    kc = torch.full((n_slots, G, cap, hd), 3.0, device=DEV, dtype=dt)
    vc = torch.full_like(kc, 3.0)
    table = None
    if paged:
        kc, vc, table = _paged(kc, vc, seed=hd + cap)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    hist = {s: [] for s in slots}
    for lens in ([150, 1, 70, 0], [300, 130, 256, 65], [240, 64, 1, 200]):
        live = [(n, s) for n, s in zip(lens, slots) if n > 0]
        b = B([n for n, _ in live], [s for _, s in live])
        N = b.n_tokens
        qkv = torch.randn(N, (H + 2 * G) * hd, device=DEV)
        q_out = torch.empty(N, H * hd, device=DEV, dtype=dt)
        kv_step = torch.empty(N, 2, G, hd, device=DEV, dtype=dt)
        ops.rope_store(qkv, 1, inv, b, q_out, kv_step, kc, vc, slot_pos, H, G, hd, cap, pages=table)
        out = torch.full((N, H * hd), 9.0, device=DEV, dtype=dt)
        ops.attention_prefill_tc_cache(q_out, kc, vc, b, slot_pos, out, H, G, hd, cap, window, status,
                                       pages=table)
        torch.cuda.synchronize()
        assert status.item() == 0
        qs = b.q_start.tolist()
        for i, (n, s) in enumerate(live):
            hist[s].append(qkv[qs[i]:qs[i + 1]].cpu().view(-1, H + 2 * G, hd))
            allt = torch.cat(hist[s])
            T = allt.shape[0]
            pos = torch.arange(T)
            qq = plain_rope(allt[:, :H], pos, inv.cpu()).to(dt).float()
            kk = plain_rope(allt[:, H:H + G], pos, inv.cpu()).to(dt).float()
            vv = allt[:, H + G:].to(dt).float()
            ref = plain_attention(qq, kk, vv, window)[T - n:]
            got = out[qs[i]:qs[i + 1]].float().cpu().view(-1, H, hd)
            assert (got - ref).abs().max().item() <= 6.4 * eps, (lens, i)
        ops.advance(b, slot_pos)


def _paged(kc, vc, seed):
    """The same cache as pages of 64 positions in a shuffled pool: (k pages, v pages, table)."""
    n_slots, G, cap, hd = kc.shape
    pps = -(-cap // 64)
    n_pages = n_slots * pps + 3
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g)[:n_slots * pps].reshape(n_slots, pps)
    kp = torch.full((G, n_pages, 64, hd), 5.0, device=DEV, dtype=kc.dtype)
    vp = torch.full_like(kp, 5.0)
    for s in range(n_slots):
        for p in range(pps):
            n = min(64, cap - p * 64)
            kp[:, perm[s, p], :n] = kc[s, :, p * 64:p * 64 + n]
            vp[:, perm[s, p], :n] = vc[s, :, p * 64:p * 64 + n]
    return kp, vp, perm.to(torch.int32).to(DEV).contiguous()


def _unpaged(kp, table, cap):
    n_slots, pps = table.shape
    out = torch.cat([kp[:, table[s].long()].reshape(1, kp.shape[0], pps * 64, kp.shape[3])
                     for s in range(n_slots)])
    return out[:, :, :cap]


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("H, G, hd, cap, window", [(8, 2, 128, 300, None), (6, 3, 48, 100, 100),
                                                   (4, 4, 16, 70, 33)])
def test_every_cache_kernel_reads_and_writes_pages_like_rows(ops, dt, H, G, hd, cap, window):
    """A cache of shuffled 64-position pages behind a page table gives, bit for bit, what
    the same rows give as one block per sequence: rotary write, ring write, and the four
    attention kernels (prompts on top of a cache, decode; SIMT and tensor cores)."""
    from plain_model import plain_inv_freq
    inv = plain_inv_freq(hd, 10000.0, None).to(DEV)
    n_slots, slots = 4, [2, 0, 3]
    g = torch.Generator(device=DEV).manual_seed(cap + hd)
    kc = torch.randn(n_slots, G, cap, hd, device=DEV, generator=g).to(dt)
    vc = torch.randn(n_slots, G, cap, hd, device=DEV, generator=g).to(dt)
    kp, vp, table = _paged(kc, vc, 3)
    past = [cap - 5, 17, 64] if window else [cap - 40, 17, 64]
    slot_pos = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
    for s, p in zip(slots, past):
        slot_pos[s] = p
    lens = [30, 1, 9] if window else [35, 1, 9]
    b = B(lens, slots)
    N = b.n_tokens
    qkv = torch.randn(N, (H + 2 * G) * hd, device=DEV, generator=g)
    outs = []
    for paged in (False, True):
        K, V, pg = (kp.clone(), vp.clone(), table) if paged else (kc.clone(), vc.clone(), None)
        q = torch.empty(N, H * hd, device=DEV, dtype=dt)
        kv = torch.empty(N, 2, G, hd, device=DEV, dtype=dt)
        ops.rope_store(qkv, 1, inv, b, q, kv, K, V, slot_pos, H, G, hd, cap, write_cache=False, pages=pg)
        res = []
        o = torch.empty(N, H * hd, device=DEV, dtype=dt)
        ops.attention(q, kv, K, V, b, slot_pos, o, H, G, hd, cap, window, 1, pages=pg)
        res.append(o.clone())
        if ops.mma_attention_usable(dt, hd):
            o2 = torch.empty_like(o)
            ops.attention_prefill_mma(q, kv, K, V, b, slot_pos, o2, H, G, hd, cap, window, pages=pg)
            res.append(o2)
        ops.cache_write(kv, b, K, V, slot_pos, G, hd, cap, pages=pg)          # the late ring write
        K2, V2 = K.clone(), V.clone()
        ops.rope_store(qkv, 1, inv, b, q, kv, K2, V2, slot_pos, H, G, hd, cap, pages=pg)
        res += [(_unpaged(K, table, cap) if paged else K), (_unpaged(K2, table, cap) if paged else K2),
                (_unpaged(V2, table, cap) if paged else V2)]
        # decode: one more token per sequence on top of what is now cached
        sp = slot_pos.clone()
        for s, p, n in zip(slots, past, lens):
            sp[s] = p + n - 1                                                  # the newest row is cached
        bd = B([1, 1, 1], slots)
        qd = torch.randn(3, H * hd, device=DEV, generator=torch.Generator(device=DEV).manual_seed(1)).to(dt)
        bound = max(p + n for p, n in zip(past, lens))
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        chunk = 32
        mc = -(-(min(bound, window) if window else bound) // chunk)
        od = torch.empty(3, H * hd, device=DEV, dtype=dt)
        ops.attention_decode(qd, K2, V2, bd.seq_slot, sp, od, torch.empty(3 * H * mc * hd, device=DEV),
                             torch.empty(3 * H * mc * 2, device=DEV),
                             torch.zeros(3 * G * -(-(H // G) // 4), dtype=torch.int32, device=DEV), status,
                             H, G, hd, cap, window, chunk, bound, pages=pg)
        res.append(od)
        if ops.mma_attention_usable(dt, hd):
            for cpc, warps in ((1, 4), (1000, 4), (1, 2), (1000, 2)):
                mp = ops.decode_mma_parts(bound, window, cpc)
                om = torch.empty(3, H * hd, device=DEV, dtype=dt)
                ops.attention_decode_mma(qd, K2, V2, bd.seq_slot, sp, om, torch.empty(3 * H * mp * hd, device=DEV),
                                         torch.empty(3 * H * mp * 2, device=DEV),
                                         torch.zeros(3 * G * -(-(H // G) // 16), dtype=torch.int32, device=DEV),
                                         status, H, G, hd, cap, window, bound, cpc, pages=pg, warps=warps)
                res.append(om)
        torch.cuda.synchronize()
        assert status.item() == 0
        outs.append(res)
    assert len(outs[0]) == len(outs[1])
    for i, (a, c) in enumerate(zip(*outs)):
        assert torch.equal(a, c), i


@pytest.mark.parametrize("dt, eps", HALF)
@pytest.mark.parametrize("H, G, hd, lens", [(4, 2, 128, [300, 1, 150]), (6, 2, 64, [129]), (5, 1, 32, [200, 260]),
                                            (3, 3, 16, [700])])
def test_many_token_product_with_rotary_epilogue(ops, H, G, hd, lens, dt, eps):
    """gemm_2sm_rope against the two-SM product followed by the rotary kernel, bit for bit:
    ragged prompts on top of filled slots, a ring that wraps, a paged cache."""
    from plain_model import plain_inv_freq
    D, cap, n_slots = 192, 96, 4
    N = (H + 2 * G) * hd
    inv = plain_inv_freq(hd, 10000.0, None).to(DEV)
    slots = [2, 0, 3][:len(lens)]
    b = B(lens, slots)
    M = b.n_tokens
    slot_pos = torch.tensor([30, 0, 70, 5], dtype=torch.int32, device=DEV)
    a = torch.randn(M, D, device=DEV).to(dt)
    w = (torch.randn(N, D, device=DEV) * 0.1).to(dt)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kc0 = torch.full((n_slots, G, cap, hd), 3.0, device=DEV, dtype=dt)
    kp0, vp0, table = _paged(kc0, kc0, 5)
    for pages in (None, table):
        for write_cache in (True, False):
            def fresh():
                kc = (kp0 if pages is not None else kc0).clone()
                return [torch.zeros(M, H * hd, device=DEV, dtype=dt), torch.zeros(M, 2, G, hd, device=DEV, dtype=dt),
                        kc, kc.clone()]
            want, got = fresh(), fresh()
            full = torch.empty(M, N, device=DEV)
            ops.gemm_2sm(a, w, full, ops.GEMM_STORE, status)
            ops.rope_store(full, 1, inv, b, want[0], want[1], want[2], want[3], slot_pos, H, G, hd, cap,
                           write_cache=write_cache, pages=pages)
            table = torch.empty(M, hd // 2, 2, device=DEV)
            ops.rope_table(inv, b, slot_pos, table)
            ops.gemm_2sm_rope(a, w, table, b, got[0], got[1], got[2], got[3], slot_pos, H, G, hd, cap, status,
                              write_cache=write_cache, pages=pages)
            torch.cuda.synchronize()
            assert status.item() == 0
            for i, (g_, w_) in enumerate(zip(got, want)):
                assert torch.equal(g_, w_), (i, write_cache, pages is not None)
