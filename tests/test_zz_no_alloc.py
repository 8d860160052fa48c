"""The allocation-free C entry point of paged decode attention (``astrai_b200_paged_decode_noalloc``).

Some hosts of this library cannot allocate GPU memory when they call into it: an inference server whose own pool
already holds the whole device, or a process that bans the CUDA allocator after start-up.  For them the library
exports one plain-C function whose scratch lives in a fixed ``__device__`` array inside the shared object.  The
test loads the exported symbol with ``ctypes`` (no torch binding in between), runs it twice in a row on the same
inputs - the second call reuses whatever the first left in the shared scratch - and compares each result with
the regular torch op, which takes caller-allocated scratch tensors, and with a plain fp32 PyTorch statement of
decode attention.  It also checks what the entry point is for: the free device memory reported by the driver is the
same before and after a call (nothing was allocated), and a sequence length larger than the table row is cut to the
row instead of reading past it.

This file sorts last so that a run that stops at the first failure has already run every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbols():
    from astrai_b200.ops import native

    native.require()
    lib = ctypes.CDLL(str(native.lib_path()))
    fn = lib.astrai_b200_paged_decode_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 5 + [ctypes.c_longlong, ctypes.c_longlong, ctypes.c_float,
                                                                 ctypes.c_void_p]
    err = lib.astrai_b200_noalloc_error
    err.restype = ctypes.c_char_p
    return fn, err


def _case(hd, hq, hkv, lens, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    b, page, max_ctx, n_slots = len(lens), 16, 1536, 4096
    k_buf = torch.randn(n_slots, hkv, hd, device="cuda", dtype=torch.bfloat16, generator=g)
    v_buf = torch.randn(n_slots, hkv, hd, device="cuda", dtype=torch.bfloat16, generator=g)
    table = torch.zeros(b, max_ctx, dtype=torch.int32, device="cuda")
    perm = torch.randperm(n_slots // page, device="cuda", generator=g)
    used = 0
    for i, n in enumerate(lens):
        pages = perm[used:used + -(-n // page)]
        used += pages.numel()
        table[i, :n] = (pages[:, None] * page + torch.arange(page, device="cuda")[None]).reshape(-1)[:n].int()
    rows = torch.arange(b, dtype=torch.int32, device="cuda")
    q = torch.randn(b, hq, hd, device="cuda", dtype=torch.bfloat16, generator=g)
    seq = torch.tensor(lens, dtype=torch.long, device="cuda")
    return q, k_buf, v_buf, table, rows, seq


def _regular(q, k_buf, v_buf, table, rows, seq, splits):
    b, hq, hd = q.shape
    hkv = k_buf.shape[1]
    o_part = torch.zeros(b, hq, 8, hd, device="cuda")
    ml_part = torch.zeros(b, hq, 8, 2, device="cuda")
    counters = torch.zeros(b * hkv, dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    torch.ops.astrai_b200.paged_decode_(q, k_buf, v_buf, table, rows, seq, hd ** -0.5, splits, o_part, ml_part, counters, out)
    return out


def _fp32_statement(q, k_buf, v_buf, table, rows, seq):
    """softmax(q k^T / sqrt(d)) v over each request's cached tokens, in fp32, one request at a time."""
    b, hq, hd = q.shape
    hkv = k_buf.shape[1]
    out = torch.zeros(b, hq, hd, device=q.device)
    for i in range(b):
        n = min(int(seq[i]), table.shape[1])
        slots = table[int(rows[i]), :n].long()
        k = k_buf[slots].float().repeat_interleave(hq // hkv, dim=1)  # [n, hq, hd]
        v = v_buf[slots].float().repeat_interleave(hq // hkv, dim=1)
        p = torch.softmax(torch.einsum("hd,nhd->hn", q[i].float(), k) * hd ** -0.5, dim=-1)
        out[i] = torch.einsum("hn,nhd->hd", p, v)
    return out


@pytest.mark.parametrize("hd,hq,hkv,lens", [(128, 16, 4, [1400, 37, 512]), (64, 8, 8, [300, 1])])
def test_noalloc_entry_matches_regular_entry_twice(hd, hq, hkv, lens):
    fn, err = _symbols()
    for call, seed in enumerate((21, 22)):  # two calls in a row share the built-in scratch
        q, k_buf, v_buf, table, rows, seq = _case(hd, hq, hkv, lens, seed)
        out = torch.full_like(q, float("nan"))
        stream = torch.cuda.current_stream().cuda_stream
        rc = fn(q.data_ptr(), k_buf.data_ptr(), v_buf.data_ptr(), table.data_ptr(), rows.data_ptr(), seq.data_ptr(),
                out.data_ptr(), len(lens), hq, hkv, hd, table.shape[1], k_buf.shape[0], max(lens), hd ** -0.5, stream)
        assert rc == 0, err().decode()
        splits = int(torch.ops.astrai_b200.paged_decode_splits(len(lens), hkv, max(lens), 8))
        ref = _regular(q, k_buf, v_buf, table, rows, seq, splits)
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all(), call
        assert (out.float() - ref.float()).abs().max().item() < 2e-2, call
        assert (out.float() - _fp32_statement(q, k_buf, v_buf, table, rows, seq)).abs().max().item() < 2e-2, call


def test_noalloc_entry_leaves_free_memory_unchanged():
    fn, err = _symbols()
    q, k_buf, v_buf, table, rows, seq = _case(128, 16, 4, [900, 64], 31)
    out = torch.empty_like(q)
    stream = torch.cuda.current_stream().cuda_stream
    args = (q.data_ptr(), k_buf.data_ptr(), v_buf.data_ptr(), table.data_ptr(), rows.data_ptr(), seq.data_ptr(),
            out.data_ptr(), 2, 16, 4, 128, table.shape[1], k_buf.shape[0], 900, 128 ** -0.5, stream)
    assert fn(*args) == 0, err().decode()  # the first call on a device resolves the scratch address
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    assert fn(*args) == 0, err().decode()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before  # the driver handed out nothing during the call


def test_length_beyond_the_table_row_is_cut_to_the_row():
    fn, err = _symbols()
    q, k_buf, v_buf, table, rows, seq = _case(128, 16, 4, [1536, 40], 32)  # request 0 fills its whole row
    too_long = seq.clone()
    too_long[0] = 5000  # claims more tokens than a row holds
    out = torch.full_like(q, float("nan"))
    rc = fn(q.data_ptr(), k_buf.data_ptr(), v_buf.data_ptr(), table.data_ptr(), rows.data_ptr(), too_long.data_ptr(),
            out.data_ptr(), 2, 16, 4, 128, table.shape[1], k_buf.shape[0], 5000, 128 ** -0.5,
            torch.cuda.current_stream().cuda_stream)
    assert rc == 0, err().decode()
    torch.cuda.synchronize()
    assert (out.float() - _fp32_statement(q, k_buf, v_buf, table, rows, seq)).abs().max().item() < 2e-2


def test_noalloc_entry_rejects_oversize():
    fn, err = _symbols()
    q, k_buf, v_buf, table, rows, seq = _case(128, 16, 4, [8], 23)
    out = torch.empty_like(q)
    # 128 requests x 16 heads x 128 dims is twice the built-in scratch: refused before any launch
    rc = fn(q.data_ptr(), k_buf.data_ptr(), v_buf.data_ptr(), table.data_ptr(), rows.data_ptr(), seq.data_ptr(),
            out.data_ptr(), 128, 16, 4, 128, table.shape[1], k_buf.shape[0], 8, 0.1, None)
    assert rc == -5 and b"exceeds the built-in scratch" in err()
    rc = fn(q.data_ptr(), k_buf.data_ptr(), v_buf.data_ptr(), table.data_ptr(), rows.data_ptr(), seq.data_ptr(),
            out.data_ptr(), 1, 16, 4, 96, table.shape[1], k_buf.shape[0], 8, 0.1, None)
    assert rc == -3
