"""Typed Python entry points of the CUDA kernels.

Each function checks device, dtype, shape and contiguity of its tensors, then calls
the C entry point with raw pointers on torch's current stream.  Outputs are written
into tensors the caller passes: nothing here allocates, so every call can be
recorded in a CUDA graph.  (The reference performs the same checks in C++,
model/kernels/csrc/ops.cpp:29-72.)
"""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from .library import KernelError, check, library

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported; float32 and bfloat16 are") from None


def _ptr(t: Optional[torch.Tensor]):
    """The tensor's device address as ctypes takes it for a pointer argument (an int; None = null)."""
    return None if t is None else t.data_ptr()


_scoped_stream = None      # the stream handle inside a stream_scope, else None


class stream_scope:
    """Inside the scope every kernel of this module goes to the stream that was current when the
    scope was entered, looked up once.  `torch.cuda.current_stream()` costs several microseconds a
    call, which with some 330 launches was a quarter of the host's time for a step; a step's
    kernels all go to one stream anyway.  The caller must not switch streams inside the scope."""

    def __enter__(self):
        global _scoped_stream
        self._outer = _scoped_stream
        _scoped_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self._outer
        return False


def _stream():
    return _scoped_stream if _scoped_stream is not None else torch.cuda.current_stream().cuda_stream


def set_dependent_launch(on: bool) -> None:
    """Whether the kernels launched from now on carry the programmatic-stream-serialization attribute (they
    may start while their predecessor in the stream still runs).  SOCRATES_PDL=0 keeps it off regardless."""
    library().sb_set_dependent_launch(int(bool(on)))


def _want(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if shape is not None and t.shape != shape:              # torch.Size compares with tuples
        raise KernelError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


def embed(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor,
          feedback: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """out[n, :] = float32(table[ids[n], :]) * scale; out float32 [N, d], ids int32 [N].
    With `feedback` (int32, on the device) an id -1 - j stands for feedback[j]: a token that an
    earlier kernel on the stream wrote."""
    V, d = table.shape
    N = ids.numel()
    _want(table, "table")
    _want(ids, "ids", torch.int32)
    _want(out, "out", torch.float32, (N, d))
    if feedback is not None:
        _want(feedback, "feedback", torch.int32)
    lib = library()
    check(lib, lib.sb_embed(_ptr(out), _ptr(table), _ptr(ids), N, d, V, _code(table.dtype), _ptr(feedback),
                            float(scale), _stream()), "embed")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor,
                out: torch.Tensor, eps: float, row_index: Optional[torch.Tensor] = None) -> None:
    """residual += sum(delta, 0); out = rmsnorm(residual) * gain.

    residual float32 [N, d]; delta float32 [S, N, d] or None; gain float32 [d];
    out [M, d] in the model dtype, M = len(row_index) or N.  With row_index only the
    named rows are normed and the residual is left as it is.
    """
    N, d = residual.shape
    _want(residual, "residual", torch.float32)
    _want(gain, "gain", torch.float32, (d,))
    S, stride = 0, 0
    if delta is not None:
        _want(delta, "delta", torch.float32)
        if delta.dim() != 3 or delta.shape[1:] != (N, d):
            raise KernelError(f"delta must be [S, {N}, {d}], got {tuple(delta.shape)}")
        S, stride = delta.shape[0], N * d
    M = N
    if row_index is not None:
        _want(row_index, "row_index", torch.int32)
        M = row_index.numel()
    _want(out, "out", None, (M, d))
    lib = library()
    check(lib, lib.sb_add_rmsnorm(_ptr(residual), _ptr(delta), S, stride, _ptr(gain), _ptr(out),
                                  _ptr(row_index), M, d, float(eps), _code(out.dtype), _stream()),
          "add_rmsnorm")


def qk_norm_rope_kvwrite(qkv: torch.Tensor, q_out: torch.Tensor, k_pool: Optional[torch.Tensor],
                         v_pool: Optional[torch.Tensor], q_gain: Optional[torch.Tensor],
                         k_gain: Optional[torch.Tensor], inv_freq: torch.Tensor, rotary_dim: int,
                         positions: torch.Tensor, token_rows: torch.Tensor, block_table: torch.Tensor,
                         eps: float, num_heads: int, num_kv_heads: int, head_dim: int,
                         value_dim: Optional[int] = None, row_width: Optional[int] = None,
                         neighbours: bool = False, bias: Optional[torch.Tensor] = None,
                         map_dim: Optional[int] = None, magnitude: float = 1.0, spread_maps: bool = False) -> None:
    """Per-head norm, rotation and paged KV write for N tokens.

    qkv [N, (Hq+2Hkv)*D] in the model dtype, or float32 [S, N, (Hq+2Hkv)*D] partial sums
    of a split product (added here); q_out [N, Hq*D]; pools [pages, Hkv, BS, D] (None:
    the keys and values of this step are not stored, the layer reads another layer's cache).
    `value_dim`: value heads of another size Dv (v_pool [pages, Hkv, BS, Dv]); `row_width`: the
    rows of qkv are wider than the heads (more columns of the same product follow them; without
    pools only the Hq query heads need be there); `neighbours`: dim 2j rotates with dim 2j+1
    instead of dim j with dim j + rotary_dim/2.  `bias`: float32 [row_width], added to the input
    columns first.  `map_dim`: a query or key head holds head_dim / map_dim maps, each of which
    rotates its own first rotary_dim dims.  `magnitude` multiplies every cosine and sine.
    `spread_maps`: q_out is [N, Hq * maps, head_dim], a row per (head, map) that holds the map's dims in
    their place and zeros elsewhere, so that a dot product with a whole key row gives that map's score.
    """
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    Dv = D if value_dim is None else int(value_dim)
    width = (Hq + Hkv) * D + Hkv * Dv if row_width is None else int(row_width)
    parts = qkv.dim() == 3
    N = qkv.shape[-2]
    if parts:
        _want(qkv, "qkv partial sums", torch.float32, (qkv.shape[0], N, width))
    else:
        _want(qkv, "qkv", q_out.dtype, (N, width))
    maps_out = (D // int(map_dim)) if (spread_maps and map_dim) else 1
    _want(q_out, "q_out", None, (N, Hq * D * maps_out))
    _want(positions, "positions", torch.int32, (N,))
    _want(token_rows, "token_rows", torch.int32, (N,))
    _want(block_table, "block_table", torch.int32)
    _want(inv_freq, "inv_freq", torch.float32)
    if inv_freq.numel() < rotary_dim // 2:
        raise KernelError(f"inv_freq has {inv_freq.numel()} entries for rotary_dim {rotary_dim}")
    write_kv = k_pool is not None
    page_size = 1
    if write_kv:
        _want(k_pool, "k_pool", q_out.dtype)
        if k_pool.dim() != 4 or k_pool.shape[1] != Hkv or k_pool.shape[3] != D:
            raise KernelError(f"pools must be [pages, {Hkv}, page_size, {D}], got {tuple(k_pool.shape)}")
        _want(v_pool, "v_pool", q_out.dtype, (*k_pool.shape[:3], Dv))
        page_size = k_pool.shape[2]
    for g, nm in ((q_gain, "q_gain"), (k_gain, "k_gain")):
        if g is not None:
            _want(g, nm, torch.float32, (D,))
    if bias is not None:
        _want(bias, "bias", torch.float32, (width,))
    sub = D if map_dim is None else int(map_dim)
    if sub < 1 or D % sub or rotary_dim > sub:
        raise KernelError(f"heads of {D} dims do not hold maps of {sub} dims with {rotary_dim} rotating")
    lib = library()
    check(lib, lib.sb_qk_norm_rope_kvwrite(
        None if parts else _ptr(qkv), _ptr(qkv) if parts else None, qkv.shape[0] if parts else 0,
        N * width, _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(q_gain), _ptr(k_gain), _ptr(inv_freq),
        rotary_dim, _ptr(positions), _ptr(token_rows), _ptr(block_table), block_table.shape[1],
        page_size, float(eps), Hq, Hkv, D, N, int(write_kv), _code(q_out.dtype), Dv, width, int(neighbours),
        _ptr(bias), sub, float(magnitude), int(bool(spread_maps)), _stream()), "qk_norm_rope_kvwrite")


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor, interleaved: bool = False) -> None:
    """out[n, f] = up * silu(gate) with gate = gate_up[n, f], up = gate_up[n, F + f], or, when
    `interleaved`, gate = gate_up[n, 2f], up = gate_up[n, 2f + 1]."""
    N, F2 = gate_up.shape
    _want(gate_up, "gate_up")
    _want(out, "out", gate_up.dtype, (N, F2 // 2))
    lib = library()
    check(lib, lib.sb_silu_mul(_ptr(out), _ptr(gate_up), N, F2 // 2, int(interleaved), _code(out.dtype), _stream()),
          "silu_mul")


def sample_scratch_size(M: int, V: int) -> int:
    """int32 entries of scratch that `sample` needs for M rows of V logits."""
    return M * (2 * library().sb_sample_slices(int(V)) + 1)


def sample(out: torch.Tensor, logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           seeds: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None,
           scratch: Optional[torch.Tensor] = None) -> None:
    """out[m] = argmax(logits[m]) where temperature[m] == 0 (or temperature is None),
    else a draw from softmax(logits[m] / temperature[m]) fixed by (seeds[m], counters[m]).

    `scratch`: int32 with at least sample_scratch_size(M, V) entries that were zero before
    its first use (the kernel leaves it ready for the next call); allocated here if None.
    """
    M, V = logits.shape
    _want(logits, "logits", torch.float32)
    _want(out, "out", torch.int32, (M,))
    if temperature is not None:
        _want(temperature, "temperature", torch.float32, (M,))
        _want(seeds, "seeds", torch.int32, (M,))
        _want(counters, "counters", torch.int32, (M,))
    need = sample_scratch_size(M, V)
    if scratch is None:
        scratch = torch.zeros(need, dtype=torch.int32, device=logits.device)
    _want(scratch, "scratch", torch.int32)
    if scratch.numel() < need:
        raise KernelError(f"sample scratch has {scratch.numel()} entries, {need} are needed")
    lib = library()
    check(lib, lib.sb_sample(_ptr(out), _ptr(logits), _ptr(temperature), _ptr(seeds), _ptr(counters),
                             M, V, _ptr(scratch), _stream()), "sample")


def gemm_simt(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, splits: int = 1) -> None:
    """out = a @ w.T on the CUDA cores with float32 accumulation.

    a [M, K], w [N, K]; out [M, N], or float32 [splits, M, N] partial sums.
    """
    M, K = a.shape
    N = w.shape[0]
    _want(a, "a")
    _want(w, "w", None, (N, K))
    if splits == 1 and out.dim() == 2:
        _want(out, "out", None, (M, N))
    else:
        _want(out, "out", torch.float32, (splits, M, N))
    lib = library()
    check(lib, lib.sb_gemm_simt(_ptr(out), _ptr(a), _ptr(w), M, N, K, _code(a.dtype), _code(w.dtype),
                                _code(out.dtype), splits, _stream()), "gemm_simt")


def attention_simt(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                   block_table: torch.Tensor, token_rows: torch.Tensor, positions: torch.Tensor,
                   num_heads: int, scale: float, window: int = 0, num_partitions: int = 1,
                   part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None) -> None:
    """Paged causal attention, one query per token, on the CUDA cores.

    q, out [N, Hq*D]; pools [pages, Hkv, BS, D]; block_table int32 [rows, W];
    window 0 = all keys.  Scratch for num_partitions > 1: part_o float32 with at least
    N*Hq*NP*D elements, part_ml with N*Hq*NP*2.
    """
    N = q.shape[0]
    pages, Hkv, BS, D = k_pool.shape
    Hq = num_heads
    _want(q, "q", k_pool.dtype, (N, Hq * D))
    _want(out, "out", q.dtype, (N, Hq * D))
    _want(k_pool, "k_pool")
    _want(v_pool, "v_pool", k_pool.dtype, k_pool.shape)
    _want(block_table, "block_table", torch.int32)
    _want(token_rows, "token_rows", torch.int32, (N,))
    _want(positions, "positions", torch.int32, (N,))
    if num_partitions > 1:
        _want(part_o, "part_o", torch.float32)
        _want(part_ml, "part_ml", torch.float32)
        if part_o.numel() < N * Hq * num_partitions * D or part_ml.numel() < N * Hq * num_partitions * 2:
            raise KernelError("attention scratch buffers are too small")
    lib = library()
    check(lib, lib.sb_attention_simt(
        _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
        block_table.shape[1], _ptr(token_rows), _ptr(positions), N, Hq, Hkv, D, BS, int(window),
        float(scale), num_partitions, _code(q.dtype), _stream()), "attention",
        kernels=2 if num_partitions > 1 else 1)


def gemm_tcgen05_splits(K: int, splits: int) -> int:
    """How many K parts `gemm_tcgen05` writes when `splits` are asked for (never more)."""
    return library().sb_gemm_tcgen05_splits(int(K), int(splits))


SHARES_VARIANT = 2000      # gemm_tcgen05 variant: the pair kernel dealing equal shares of K blocks


def gemm_tcgen05_shares_parts(M: int, N: int, K: int) -> int:
    """How many float32 parts `gemm_tcgen05(..., variant=SHARES_VARIANT)` writes for this shape: the
    pair kernel (two SMs per 256 x 256 tile) with the tiles' K blocks dealt to the pairs in equal
    shares, a tile that a share's end cuts being finished by the next pair into another part.
    0: the shape is not served (few rows, N below 256, more than four pieces to a tile)."""
    return int(library().sb_gemm_tcgen05_shares_parts(int(M), int(N), int(K)))


def gemm_tcgen05(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, status: torch.Tensor,
                 splits: int = 1, variant: int = 0, epilogue: int = 0,
                 prefetch: Optional[Tuple[torch.Tensor, int]] = None) -> int:
    """out = a @ w.T on the tcgen05 tensor cores; a [M, K] and w [N, K] bfloat16, K % 8 == 0.

    out is bfloat16 or float32 [M, N], or float32 [S, M, N] partial sums where S =
    gemm_tcgen05_splits(K, splits).  `status` is an int32 device tensor that receives a
    non-zero code if a bounded wait inside the kernel gave up.  Returns S.
    `prefetch`: (tensor, bytes), the leading bytes of the weights that the next product
    streams; the weight-streaming kernel (M <= 64) asks for them in L2 once its own loads
    are issued.
    """
    M, K = a.shape
    N = w.shape[0]
    _want(a, "a", torch.bfloat16)
    _want(w, "w", torch.bfloat16, (N, K))
    _want(status, "status", torch.int32)
    S = gemm_tcgen05_shares_parts(M, N, K) if variant == SHARES_VARIANT else gemm_tcgen05_splits(K, splits)
    if variant == SHARES_VARIANT and (S == 0 or out.dim() != 3):
        raise KernelError(f"the equal-shares kernel does not serve M={M} N={N} K={K} (or out is not [S, M, N])")
    if out.dim() == 2:
        if S != 1:
            raise KernelError("a split product needs a float32 [S, M, N] output")
        _want(out, "out", None, (M, N // 2 if epilogue == 1 else N))
    else:
        _want(out, "out", torch.float32, (S, M, N))
    lib = library()
    s_io = ctypes.c_int(S)
    pf_ptr, pf_bytes = None, 0
    if prefetch is not None and M <= 64:
        tensor, nbytes = prefetch
        if not tensor.is_cuda or not tensor.is_contiguous():
            raise KernelError("a prefetch range must be a contiguous CUDA tensor")
        pf_ptr = tensor.data_ptr()
        pf_bytes = max(0, min(int(nbytes), tensor.numel() * tensor.element_size()))
    check(lib, lib.sb_gemm_tcgen05(_ptr(out), _ptr(a), _ptr(w), M, N, K, _code(out.dtype),
                                   ctypes.byref(s_io), _ptr(status), int(variant), int(epilogue),
                                   pf_ptr, pf_bytes, _stream()),
          "gemm_tcgen05")
    if s_io.value != S:
        raise KernelError(f"gemm_tcgen05 wrote {s_io.value} parts where {S} were expected")
    return S


def attention_mma_supports(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                           decode: bool) -> bool:
    """Whether the tensor-core attention kernels take this shape (bfloat16 only)."""
    return bool(library().sb_attention_mma_supports(num_heads, num_kv_heads, head_dim, page_size,
                                                    int(decode)))


def attention_prefill_mma(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                          block_table: torch.Tensor, seq_starts: torch.Tensor, seq_rows: torch.Tensor,
                          seq_first_pos: torch.Tensor, num_heads: int, scale: float, window: int = 0) -> None:
    """Paged causal attention of prompt portions on the tensor cores (bfloat16).

    Request r brings tokens seq_starts[r] .. seq_starts[r+1]-1 (rows of q and out) at
    positions seq_first_pos[r], +1, ... of cache row seq_rows[r]; its keys, earlier
    portions included, are read from the pages.
    """
    N = q.shape[0]
    _, Hkv, BS, D = k_pool.shape
    R = seq_rows.numel()
    _want(q, "q", torch.bfloat16, (N, num_heads * D))
    _want(out, "out", torch.bfloat16, (N, num_heads * D))
    _want(k_pool, "k_pool", torch.bfloat16)
    _want(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    _want(block_table, "block_table", torch.int32)
    _want(seq_starts, "seq_starts", torch.int32, (R + 1,))
    _want(seq_rows, "seq_rows", torch.int32, (R,))
    _want(seq_first_pos, "seq_first_pos", torch.int32, (R,))
    lib = library()
    check(lib, lib.sb_attention_prefill_mma(
        _ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
        _ptr(seq_starts), _ptr(seq_rows), _ptr(seq_first_pos), R, N, num_heads, Hkv, D, BS, int(window),
        float(scale), _stream()), "attention_prefill_mma")


def attention_decode_mma(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                         block_table: torch.Tensor, token_rows: torch.Tensor, positions: torch.Tensor,
                         num_heads: int, scale: float, window: int = 0, num_partitions: int = 1,
                         part_o: Optional[torch.Tensor] = None,
                         part_ml: Optional[torch.Tensor] = None, variant: int = 0) -> None:
    """Paged attention of single decode tokens on the tensor cores (bfloat16), the keys
    of each token cut into `num_partitions` parts; arguments as `attention_simt`.
    `variant` picks the kernel's (warps, stages); 0 is the default.  2 to 4 partitions are
    merged inside the kernel (a thread-block cluster per token and KV head), more by a
    reduce kernel through the scratch buffers.

    The kernel reads the block table, rows, positions and the keys and values below each
    position before it waits for the kernel that precedes it on the stream: those must be
    older than that kernel (a host copy, an earlier step)."""
    N = q.shape[0]
    _, Hkv, BS, D = k_pool.shape
    Hq = num_heads
    _want(q, "q", torch.bfloat16, (N, Hq * D))
    _want(out, "out", torch.bfloat16, (N, Hq * D))
    _want(k_pool, "k_pool", torch.bfloat16)
    _want(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    _want(block_table, "block_table", torch.int32)
    _want(token_rows, "token_rows", torch.int32, (N,))
    _want(positions, "positions", torch.int32, (N,))
    if num_partitions > 1:
        _want(part_o, "part_o", torch.float32)
        _want(part_ml, "part_ml", torch.float32)
        if part_o.numel() < N * Hq * num_partitions * D or part_ml.numel() < N * Hq * num_partitions * 2:
            raise KernelError("attention scratch buffers are too small")
    lib = library()
    check(lib, lib.sb_attention_decode_mma(
        _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
        block_table.shape[1], _ptr(token_rows), _ptr(positions), N, Hq, Hkv, D, BS, int(window),
        float(scale), num_partitions, int(variant), _stream()), "attention_decode_mma",
        kernels=lib.sb_attention_decode_mma_kernels(num_partitions))


def attention_decode_stream_supports(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the streaming decode kernel takes this shape (bfloat16; head sizes 16 to 128, groups
    of up to 16 query heads, pages of at least 16 slots)."""
    return bool(library().sb_attention_decode_stream_supports(num_heads, num_kv_heads, head_dim, page_size))


def attention_decode_stream(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                            block_table: torch.Tensor, token_rows: torch.Tensor, positions: torch.Tensor,
                            num_heads: int, scale: float, window: int, chunk_keys: int, max_chunks: int,
                            part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                            counters: Optional[torch.Tensor] = None, variant: int = 0) -> None:
    """Paged attention of single decode tokens (bfloat16) as one persistent kernel whose warps
    stream fixed chunks of `chunk_keys` keys (a multiple of 16) of each (token, KV head); a row's
    chunks lie at fixed key positions, so its numbers do not depend on the rest of the batch.

    `max_chunks` bounds the chunks the visible keys of any token span.  Scratch for max_chunks > 1:
    part_o float32 with N*Hq*max_chunks*D elements, part_ml with N*Hq*max_chunks*2, and int32
    `counters` with N*Hkv entries that are zero before the first call (the kernel leaves them zero).

    The kernel reads the block table, rows, positions and the keys and values below each
    position before it waits for the kernel that precedes it on the stream: those must be
    older than that kernel (a host copy, an earlier step)."""
    N = q.shape[0]
    _, Hkv, BS, D = k_pool.shape
    Hq = num_heads
    _want(q, "q", torch.bfloat16, (N, Hq * D))
    _want(out, "out", torch.bfloat16, (N, Hq * D))
    _want(k_pool, "k_pool", torch.bfloat16)
    _want(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    _want(block_table, "block_table", torch.int32)
    _want(token_rows, "token_rows", torch.int32, (N,))
    _want(positions, "positions", torch.int32, (N,))
    if max_chunks > 1:
        _want(part_o, "part_o", torch.float32)
        _want(part_ml, "part_ml", torch.float32)
        _want(counters, "counters", torch.int32)
        if (part_o.numel() < N * Hq * max_chunks * D or part_ml.numel() < N * Hq * max_chunks * 2
                or counters.numel() < N * Hkv):
            raise KernelError("attention scratch buffers are too small")
    lib = library()
    check(lib, lib.sb_attention_decode_stream(
        _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(counters), _ptr(q), _ptr(k_pool), _ptr(v_pool),
        _ptr(block_table), block_table.shape[1], _ptr(token_rows), _ptr(positions), N, Hq, Hkv, D, BS,
        int(window), float(scale), int(chunk_keys), int(max_chunks), int(variant), _stream()),
        "attention_decode_stream")


def attention_decode_mma_blocks_per_sm(head_dim: int, variant: int = 0) -> int:
    """Blocks of the decode attention kernel that are resident on one SM at a time."""
    return library().sb_attention_decode_mma_blocks_per_sm(int(head_dim), int(variant))


def attention_tcgen05_supports(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 tile kernel takes this shape (bfloat16, head_dim 64 or 128)."""
    return bool(library().sb_attention_tcgen05_supports(num_heads, num_kv_heads, head_dim, page_size))


def attention_prefill_tcgen05(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                              block_table: torch.Tensor, seq_starts: torch.Tensor, seq_rows: torch.Tensor,
                              seq_first_pos: torch.Tensor, num_heads: int, scale: float, status: torch.Tensor,
                              window: int = 0, gate: Optional[torch.Tensor] = None, gate_per_dim: bool = False,
                              sink: Optional[float] = None, keep_first: int = 0,
                              out_float: Optional[torch.Tensor] = None) -> None:
    """Paged causal attention of prompt portions on tcgen05 (scores and P.V in tensor
    memory, pages brought in by TMA).  Arguments as `attention_prefill_mma`, plus the int32
    status word that receives a non-zero code if a bounded wait inside the kernel gave up.
    `keep_first`: a window also sees the first so many keys of its row.  `out_float` (float32
    [N, Hq*D]): the rows go there unrounded instead of to `out` (which may then be None)."""
    N = q.shape[0]
    pages, Hkv, BS, D = k_pool.shape
    R = seq_rows.numel()
    _want(q, "q", torch.bfloat16, (N, num_heads * D))
    if out_float is not None:
        _want(out_float, "out_float", torch.float32, (N, num_heads * D))
        if gate is not None:
            raise KernelError("the float32 rows are written ungated")
    else:
        _want(out, "out", torch.bfloat16, (N, num_heads * D))
    _want(k_pool, "k_pool", torch.bfloat16)
    _want(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    _want(block_table, "block_table", torch.int32)
    _want(seq_starts, "seq_starts", torch.int32, (R + 1,))
    _want(seq_rows, "seq_rows", torch.int32, (R,))
    _want(seq_first_pos, "seq_first_pos", torch.int32, (R,))
    _want(status, "status", torch.int32)
    # optional: out *= sigmoid(gate) (gate [N, >= Hq] or, with gate_per_dim, [N, >= Hq*D], bfloat16) and a sink,
    # a score whose exponential joins the softmax denominator without a value
    gate_stride = _gate_stride(gate, q, N, num_heads * D if gate_per_dim else num_heads)
    lib = library()
    check(lib, lib.sb_attention_prefill_tcgen05(
        _ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), pages, _ptr(block_table), block_table.shape[1],
        _ptr(seq_starts), _ptr(seq_rows), _ptr(seq_first_pos), R, N, num_heads, Hkv, D, BS, int(window),
        float(scale), _ptr(status), _ptr(gate), gate_stride, int(gate_per_dim), int(sink is not None),
        float(sink or 0.0), int(keep_first), _ptr(out_float), _stream()), "attention_prefill_tcgen05")


# ---------------------------------------------------------------------------------------------
# Kernels of blocks that norm a branch before it joins the residual, and of recurrent mixers.

ACTIVATIONS = {"identity": 0, "relu_squared": 1, "gelu_tanh": 2, "silu": 3}


def fold_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], gain: Optional[torch.Tensor],
                 out: Optional[torch.Tensor], eps: float, row_index: Optional[torch.Tensor] = None,
                 branch_bias: Optional[torch.Tensor] = None, branch_gain: Optional[torch.Tensor] = None,
                 branch_eps: float = 0.0, add_rows: Optional[torch.Tensor] = None,
                 add_vec: Optional[torch.Tensor] = None) -> None:
    """b = sum(delta, 0) + branch_bias; with `branch_gain` b = b / sqrt(mean(b^2) + branch_eps) * branch_gain;
    residual += b + add_rows + add_vec; out = residual / sqrt(mean(residual^2) + eps) * gain
    (gain None with an out: out = residual, rounded to out's dtype).

    residual float32 [N, d]; delta float32 [S, N, d] or None; the gains, the bias and add_vec float32 [d];
    add_rows float32 [N, d]; out [M, d] in float32 or bfloat16, or None (only the residual moves on).  With
    `row_index` only the named rows are computed and the residual is left as it is.
    """
    N, d = residual.shape
    _want(residual, "residual", torch.float32)
    S, stride = 0, 0
    if delta is not None:
        _want(delta, "delta", torch.float32)
        if delta.dim() != 3 or delta.shape[1:] != (N, d):
            raise KernelError(f"delta must be [S, {N}, {d}], got {tuple(delta.shape)}")
        S, stride = delta.shape[0], N * d
    for t, nm in ((gain, "gain"), (branch_bias, "branch_bias"), (branch_gain, "branch_gain"), (add_vec, "add_vec")):
        if t is not None:
            _want(t, nm, torch.float32, (d,))
    if add_rows is not None:
        _want(add_rows, "add_rows", torch.float32, (N, d))
    M = N
    if row_index is not None:
        _want(row_index, "row_index", torch.int32)
        M = row_index.numel()
    code = 0
    if out is not None:
        _want(out, "out", None, (M, d))
        code = _code(out.dtype)
    lib = library()
    check(lib, lib.sb_fold_rmsnorm(_ptr(residual), _ptr(delta), S, stride, _ptr(branch_bias), _ptr(branch_gain),
                                   float(branch_eps), _ptr(add_rows), _ptr(add_vec), _ptr(gain), _ptr(out),
                                   _ptr(row_index), M, d, float(eps), code, _stream()), "fold_rmsnorm")


def normed_mean(out: torch.Tensor, x0: torch.Tensor, gain0: torch.Tensor, x1: torch.Tensor, gain1: torch.Tensor,
                eps: float, scale: float = 0.5) -> None:
    """out = scale * (unit_rms(sum(x0, 0)) * gain0 + unit_rms(sum(x1, 0)) * gain1); x float32 [S, N, d]
    partial sums, out float32 [N, d]."""
    N, d = out.shape
    _want(out, "out", torch.float32)
    for x, g in ((x0, gain0), (x1, gain1)):
        _want(x, "x", torch.float32)
        if x.dim() != 3 or x.shape[1:] != (N, d):
            raise KernelError(f"a term must be [S, {N}, {d}], got {tuple(x.shape)}")
        _want(g, "gain", torch.float32, (d,))
    lib = library()
    check(lib, lib.sb_normed_mean(_ptr(out), _ptr(x0), x0.shape[0], N * d, _ptr(gain0), _ptr(x1), x1.shape[0],
                                  N * d, _ptr(gain1), N, d, float(eps), float(scale), _stream()), "normed_mean")


def bias_act(out: torch.Tensor, x: torch.Tensor, bias: Optional[torch.Tensor], activation: str) -> None:
    """out = act(x + bias); x [N, F] in out's dtype, or float32 partial sums [S, N, F] that are added first."""
    N, F_ = out.shape
    _want(out, "out")
    parts = x.dim() == 3
    if parts:
        _want(x, "x partial sums", torch.float32, (x.shape[0], N, F_))
    else:
        _want(x, "x", out.dtype, (N, F_))
    if bias is not None:
        _want(bias, "bias", torch.float32, (F_,))
    lib = library()
    check(lib, lib.sb_bias_act(_ptr(out), None if parts else _ptr(x), _ptr(x) if parts else None,
                               x.shape[0] if parts else 0, N * F_, _ptr(bias), N, F_, ACTIVATIONS[activation],
                               _code(out.dtype), _stream()), "bias_act")


def short_conv(x: torch.Tensor, in_bias: Optional[torch.Tensor], taps: torch.Tensor,
               conv_bias: Optional[torch.Tensor], silu: bool, tail: Optional[torch.Tensor],
               token_rows: torch.Tensor, positions: torch.Tensor, destinations,
               block_table: Optional[torch.Tensor] = None) -> None:
    """Causal convolution over time of the first C columns of x [N, >= C], per channel.

    y_t = act(sum_j taps[:, j] * (x + in_bias)_{t-K+1+j} + conv_bias), zeros before a sequence's start; tokens
    before the step's portion come from `tail` float32 [rows, K-1, C] (not changed here: `short_conv_tail`).
    `destinations`: up to three (begin, end, tensor) column ranges; a 2-d tensor [N, end-begin] is written
    densely, a 4-d pool [pages, heads, page_size, head_dim] at each token's slot through `block_table`.
    """
    C, K = taps.shape
    N = x.shape[0]
    if x.dim() != 2 or x.shape[1] < C or x.stride(1) != 1:
        raise KernelError(f"x must be [N, >= {C}] with unit column stride, got {tuple(x.shape)}")
    if not x.is_cuda:
        raise KernelError("x must be a CUDA tensor")
    _want(taps, "taps", torch.float32)
    for t, nm in ((in_bias, "in_bias"), (conv_bias, "conv_bias")):
        if t is not None:
            _want(t, nm, torch.float32, (C,))
    if K > 1:
        _want(tail, "tail", torch.float32)
        if tail.shape[1:] != (K - 1, C):
            raise KernelError(f"tail must be [rows, {K - 1}, {C}], got {tuple(tail.shape)}")
    _want(token_rows, "token_rows", torch.int32, (N,))
    _want(positions, "positions", torch.int32, (N,))
    n = len(destinations)
    if not 1 <= n <= 3:
        raise KernelError("short_conv takes one to three destinations")
    IntArr, PtrArr, LLArr = ctypes.c_int * n, ctypes.c_void_p * n, ctypes.c_longlong * n
    begin, end, paged, dst, stride, heads, hd = IntArr(), IntArr(), IntArr(), PtrArr(), LLArr(), IntArr(), IntArr()
    page_size = 0
    for i, (b, e, t) in enumerate(destinations):
        _want(t, "destination", x.dtype)
        begin[i], end[i], dst[i] = b, e, t.data_ptr()
        if t.dim() == 2:
            if t.shape != (N, e - b):
                raise KernelError(f"a dense destination must be [{N}, {e - b}], got {tuple(t.shape)}")
            paged[i], stride[i], heads[i], hd[i] = 0, e - b, 0, 0
        elif t.dim() == 4:
            if t.shape[1] * t.shape[3] != e - b:
                raise KernelError(f"a pool of {t.shape[1]} x {t.shape[3]} does not hold {e - b} channels")
            paged[i], stride[i], heads[i], hd[i] = 1, 0, t.shape[1], t.shape[3]
            page_size = t.shape[2]
            if block_table is None:
                raise KernelError("a paged destination needs the block table")
        else:
            raise KernelError("a destination is a matrix or a pool")
    if block_table is not None:
        _want(block_table, "block_table", torch.int32)
    lib = library()
    check(lib, lib.sb_short_conv(_ptr(x), x.stride(0), _ptr(in_bias), _ptr(taps), _ptr(conv_bias), int(silu),
                                 _ptr(tail), C, K, N, _ptr(token_rows), _ptr(positions), _ptr(block_table),
                                 block_table.shape[1] if block_table is not None else 0, page_size, n, begin, end,
                                 paged, dst, stride, heads, hd, _code(x.dtype), _stream()), "short_conv")


def short_conv_tail(tail: torch.Tensor, x: torch.Tensor, in_bias: Optional[torch.Tensor], taps: int,
                    seq_starts: torch.Tensor, seq_rows: torch.Tensor) -> None:
    """Move every request's tail on: it becomes the last K-1 values of (old tail, the step's x + in_bias)."""
    if taps <= 1:
        return
    R = seq_rows.numel()
    C = tail.shape[2]
    _want(tail, "tail", torch.float32)
    if x.dim() != 2 or x.shape[1] < C or x.stride(1) != 1 or not x.is_cuda:
        raise KernelError(f"x must be a CUDA matrix [N, >= {C}] with unit column stride")
    _want(seq_starts, "seq_starts", torch.int32, (R + 1,))
    _want(seq_rows, "seq_rows", torch.int32, (R,))
    lib = library()
    check(lib, lib.sb_short_conv_tail(_ptr(tail), _ptr(x), x.stride(0), _ptr(in_bias), C, taps, _ptr(seq_starts),
                                      _ptr(seq_rows), R, _code(x.dtype), _stream()), "short_conv_tail")


def retention(out: torch.Tensor, qkvg: torch.Tensor, offsets: Tuple[int, int, int, int], state: torch.Tensor,
              decay: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, seq_starts: torch.Tensor,
              seq_rows: torch.Tensor, seq_first_pos: torch.Tensor, eps: float, k_scale: float,
              chunked: bool = False, inv_freq_lo: Optional[torch.Tensor] = None,
              scratch: Optional[torch.Tensor] = None) -> None:
    """Decayed linear attention of every request's tokens of the step, in order, through its state slot.

    qkvg [N, width] holds q, k (H x dk each), v and g (H x dv each) at the column `offsets`; state float32
    [rows, H, dk, dv] is read and left advanced; out [N, H*dv] = unit_rms(S^T q) * silu(g) per head.
    `chunked`: the kernel for prompt portions, which works on up to 64 tokens of a request at once (the same
    sums in another order); without it every token is a step of the recurrence, which is what a decode step wants.
    `inv_freq_lo`: float32, what rounding to float32 took from each frequency; the angles are then carried in two
    terms and positions in the thousands cost no accuracy.
    `scratch` (float32, `retention_scratch_size` elements): lets the chunked kernel give every chunk a block of
    its own (three launches) when the requests' heads alone would leave the GPU idle."""
    N = qkvg.shape[0]
    _, H, dk, dv = state.shape
    R = seq_rows.numel()
    _want(qkvg, "qkvg", out.dtype)
    _want(out, "out", None, (N, H * dv))
    _want(state, "state", torch.float32)
    _want(decay, "decay", torch.float32, (H,))
    _want(inv_freq, "inv_freq", torch.float32)
    if inv_freq.numel() < rotary_dim // 2:
        raise KernelError(f"inv_freq has {inv_freq.numel()} entries for rotary_dim {rotary_dim}")
    _want(seq_starts, "seq_starts", torch.int32, (R + 1,))
    _want(seq_rows, "seq_rows", torch.int32, (R,))
    _want(seq_first_pos, "seq_first_pos", torch.int32, (R,))
    if inv_freq_lo is not None:
        _want(inv_freq_lo, "inv_freq_lo", torch.float32, inv_freq.shape)
    if scratch is not None:
        _want(scratch, "scratch", torch.float32)
    lib = library()
    check(lib, lib.sb_retention(_ptr(qkvg), qkvg.stride(0), *[int(o) for o in offsets], _ptr(state), _ptr(decay),
                                _ptr(inv_freq), _ptr(inv_freq_lo), int(rotary_dim), _ptr(out), _ptr(seq_starts), _ptr(seq_rows),
                                _ptr(seq_first_pos), R, H, dk, dv, float(eps), float(k_scale), int(chunked), N,
                                _ptr(scratch), scratch.numel() if scratch is not None else 0,
                                _code(out.dtype), _stream()), "retention", kernels=3 if scratch is not None else 1)


def retention_scratch_size(N: int, R: int, H: int, dk: int, dv: int) -> int:
    """float32 elements of scratch with which `retention(chunked=True)` can spread the chunks of N tokens of R
    requests over the GPU: one state per chunk and head."""
    C = int(library().sb_retention_chunk(int(dk), int(dv)))
    return (-(-N // C) + R) * H * dk * dv if C > 0 else 0


def selective_scan(out: torch.Tensor, x: torch.Tensor, z: torch.Tensor, dt_raw: torch.Tensor,
                   dt_bias: torch.Tensor, bc: torch.Tensor, A_log: torch.Tensor, D: torch.Tensor,
                   state: torch.Tensor, seq_starts: torch.Tensor, seq_rows: torch.Tensor,
                   scratch: Optional[torch.Tensor] = None) -> None:
    """Selective scan of every request's tokens of the step, in order, through its state slot.

    x, z [N, inner] (row strides may exceed inner), bc [N, 2*states] (B then C) in out's dtype; dt_raw float32
    [N, inner] before bias and softplus; A_log float32 [inner, states]; state float32 [rows, inner, states].
    `scratch` (float32, `selective_scan_scratch_size` elements): lets few requests with long portions run as
    segments of 128 tokens in parallel (three launches: the same sums with the decays of a segment multiplied up)."""
    N, inner = out.shape
    states = A_log.shape[1]
    R = seq_rows.numel()
    _want(out, "out")
    for t, nm, cols in ((x, "x", inner), (z, "z", inner), (bc, "bc", 2 * states)):
        if t.dtype != out.dtype or t.dim() != 2 or t.shape[0] != N or t.shape[1] < cols or t.stride(1) != 1:
            raise KernelError(f"{nm} must be [{N}, >= {cols}] in {out.dtype} with unit column stride")
    _want(dt_raw, "dt_raw", torch.float32, (N, inner))
    _want(dt_bias, "dt_bias", torch.float32, (inner,))
    _want(A_log, "A_log", torch.float32, (inner, states))
    _want(D, "D", torch.float32, (inner,))
    _want(state, "state", torch.float32)
    if state.shape[1:] != (inner, states):
        raise KernelError(f"state must be [rows, {inner}, {states}], got {tuple(state.shape)}")
    _want(seq_starts, "seq_starts", torch.int32, (R + 1,))
    _want(seq_rows, "seq_rows", torch.int32, (R,))
    if scratch is not None:
        _want(scratch, "scratch", torch.float32)
    lib = library()
    check(lib, lib.sb_selective_scan(_ptr(x), x.stride(0), _ptr(z), z.stride(0), _ptr(dt_raw), _ptr(dt_bias),
                                     _ptr(bc), bc.stride(0), _ptr(A_log), _ptr(D), _ptr(state), _ptr(out),
                                     _ptr(seq_starts), _ptr(seq_rows), R, inner, states, N, _ptr(scratch),
                                     scratch.numel() if scratch is not None else 0, _code(out.dtype),
                                     _stream()), "selective_scan", kernels=3 if scratch is not None else 1)


def selective_scan_scratch_size(N: int, R: int, inner: int, states: int) -> int:
    """float32 elements of scratch for `selective_scan(..., scratch=...)` on N tokens of R requests."""
    return int(library().sb_selective_scan_scratch(int(N), int(R), int(inner), int(states)))


def _gate_stride(gate: Optional[torch.Tensor], q: torch.Tensor, N: int, columns: int) -> int:
    if gate is None:
        return 0
    if gate.dtype != q.dtype or gate.dim() != 2 or gate.shape[0] != N or gate.shape[1] < columns or gate.stride(1) != 1:
        raise KernelError(f"gate must be [{N}, >= {columns}] in {q.dtype} with unit column stride")
    return gate.stride(0)


def attention_bias(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                   block_table: torch.Tensor, token_rows: torch.Tensor, positions: torch.Tensor, num_heads: int,
                   scale: float, window: int = 0, softcap: float = 0.0,
                   dist_bias: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                   num_partitions: int = 1, part_o: Optional[torch.Tensor] = None,
                   part_ml: Optional[torch.Tensor] = None, gate_per_dim: bool = False,
                   sink: Optional[float] = None) -> None:
    """Paged causal attention, one query per token, with scores capped by softcap * tanh(s / softcap)
    (0: no cap), a float32 bias table [Hq, L] by distance (distances past L-1 use the last entry) and a
    sigmoid gate per head (gate [N, >= Hq], head h at column h).  Keys and values may have different head
    sizes: q [N, Hq*Dk], k_pool [pages, Hkv, BS, Dk], v_pool [pages, Hkv, BS, Dv], out [N, Hq*Dv].
    `gate_per_dim`: the gate is [N, >= Hq*Dv], one per head and value dim (column h*Dv + d).  `sink`: a score
    whose exponential joins the softmax denominator without a value (0.0: "one added to the denominator").
    With `num_partitions` > 1 every token's visible keys are cut into that many equal shares, one block
    each, merged by a second kernel through the float32 scratch part_o (N*Hq*NP*Dv) and part_ml (N*Hq*NP*2)."""
    N = q.shape[0]
    pages, Hkv, BS, Dk = k_pool.shape
    Dv = v_pool.shape[3]
    Hq = num_heads
    _want(q, "q", k_pool.dtype, (N, Hq * Dk))
    _want(out, "out", q.dtype, (N, Hq * Dv))
    _want(k_pool, "k_pool")
    _want(v_pool, "v_pool", k_pool.dtype, (pages, Hkv, BS, Dv))
    _want(block_table, "block_table", torch.int32)
    _want(token_rows, "token_rows", torch.int32, (N,))
    _want(positions, "positions", torch.int32, (N,))
    L = 0
    if dist_bias is not None:
        _want(dist_bias, "dist_bias", torch.float32)
        if dist_bias.dim() != 2 or dist_bias.shape[0] != Hq:
            raise KernelError(f"dist_bias must be [{Hq}, L], got {tuple(dist_bias.shape)}")
        L = dist_bias.shape[1]
    gate_stride = _gate_stride(gate, q, N, Hq * Dv if gate_per_dim else Hq)
    if num_partitions > 1:
        _want(part_o, "part_o", torch.float32)
        _want(part_ml, "part_ml", torch.float32)
        if part_o.numel() < N * Hq * num_partitions * Dv or part_ml.numel() < N * Hq * num_partitions * 2:
            raise KernelError("attention scratch buffers are too small")
    lib = library()
    check(lib, lib.sb_attention_bias(_ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                     block_table.shape[1], _ptr(token_rows), _ptr(positions), _ptr(gate), gate_stride,
                                     _ptr(dist_bias), L, N, Hq, Hkv, Dk, Dv, BS, int(window), float(scale),
                                     float(softcap), int(num_partitions), _ptr(part_o), _ptr(part_ml),
                                     _code(q.dtype), int(gate_per_dim), int(sink is not None),
                                     float(sink or 0.0), _stream()), "attention_bias",
          kernels=2 if num_partitions > 1 else 1)


def attention_bias_tile_supports(num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                                 dtype: torch.dtype) -> bool:
    """Whether the tile kernel for prompt portions takes this shape (value heads up to 128 dims, key rows
    that are whole 16-byte pieces)."""
    return bool(library().sb_attention_bias_tile_supports(num_heads, num_kv_heads, key_dim, value_dim, _code(dtype)))


def attention_bias_tile(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                        block_table: torch.Tensor, seq_starts: torch.Tensor, seq_rows: torch.Tensor,
                        seq_first_pos: torch.Tensor, num_heads: int, scale: float, window: int = 0,
                        softcap: float = 0.0, dist_bias: Optional[torch.Tensor] = None,
                        gate: Optional[torch.Tensor] = None, gate_per_dim: bool = False,
                        sink: Optional[float] = None) -> None:
    """`attention_bias` for prompt portions: request r brings tokens seq_starts[r] .. seq_starts[r+1]-1 at
    positions seq_first_pos[r], +1, ... of cache row seq_rows[r]; a block serves a tile of consecutive tokens
    of one request, so a key or value row fetched once serves all of them.  The same arithmetic in float32."""
    N = q.shape[0]
    pages, Hkv, BS, Dk = k_pool.shape
    Dv = v_pool.shape[3]
    Hq = num_heads
    R = seq_rows.numel()
    _want(q, "q", k_pool.dtype, (N, Hq * Dk))
    _want(out, "out", q.dtype, (N, Hq * Dv))
    _want(k_pool, "k_pool")
    _want(v_pool, "v_pool", k_pool.dtype, (pages, Hkv, BS, Dv))
    _want(block_table, "block_table", torch.int32)
    _want(seq_starts, "seq_starts", torch.int32, (R + 1,))
    _want(seq_rows, "seq_rows", torch.int32, (R,))
    _want(seq_first_pos, "seq_first_pos", torch.int32, (R,))
    L = 0
    if dist_bias is not None:
        _want(dist_bias, "dist_bias", torch.float32)
        if dist_bias.dim() != 2 or dist_bias.shape[0] != Hq:
            raise KernelError(f"dist_bias must be [{Hq}, L], got {tuple(dist_bias.shape)}")
        L = dist_bias.shape[1]
    gate_stride = _gate_stride(gate, q, N, Hq * Dv if gate_per_dim else Hq)
    lib = library()
    check(lib, lib.sb_attention_bias_tile(_ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                          block_table.shape[1], _ptr(seq_starts), _ptr(seq_rows), _ptr(seq_first_pos),
                                          R, _ptr(gate), gate_stride, _ptr(dist_bias), L, N, Hq, Hkv, Dk, Dv, BS,
                                          int(window), float(scale), float(softcap), _code(q.dtype),
                                          int(gate_per_dim), int(sink is not None), float(sink or 0.0), _stream()),
          "attention_bias_tile")


# Gated delta rule and the routing of a mixture of experts.

def delta_rule_supports(key_dim: int, value_dim: int) -> bool:
    """Whether the delta-rule kernel takes heads of these sizes (keys up to 256 dims, values up to 1,024)."""
    return bool(library().sb_delta_rule_supports(int(key_dim), int(value_dim)))


def delta_rule(out: torch.Tensor, qkv: torch.Tensor, offsets: Tuple[int, int, int], proj: torch.Tensor,
               proj_offsets: Tuple[int, int, int], A_log: torch.Tensor, dt_bias: torch.Tensor, norm_w: torch.Tensor,
               state: torch.Tensor, seq_starts: torch.Tensor, seq_rows: torch.Tensor, num_heads: int,
               num_key_heads: int, key_dim: int, value_dim: int, eps: float, q_scale: float,
               scratch: Optional[torch.Tensor] = None) -> None:
    """The gated delta rule over the tokens of a step, request by request, token by token.

    qkv [N, >=] holds q and k (G heads of D dims, at columns offsets[0], offsets[1]) and v (H heads of Dv, at
    offsets[2]) after their convolutions and activations; proj [N, >=] the output gate (H*Dv columns at
    proj_offsets[0]), the write strength b and the decay input a (H columns each at proj_offsets[1], [2]).
    Per head: q, k become unit vectors (q times q_scale), beta = sigmoid(b), g = exp(-exp(A_log) *
    softplus(a + dt_bias)); S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; out = o / rms(o) *
    norm_w * silu(gate).  state float32 [rows, H, D, Dv] is read and left for the next step.  `scratch`:
    float32, at least N*H*Dv elements (o before the norm; allocated here when it is not given, which a step
    that may be recorded into a graph must not rely on)."""
    N = out.shape[0]
    H, G, D, Dv = int(num_heads), int(num_key_heads), int(key_dim), int(value_dim)
    R = seq_rows.numel()
    _want(out, "out", None, (N, H * Dv))
    for t, nm in ((qkv, "qkv"), (proj, "proj")):
        if t.dim() != 2 or t.shape[0] != N or t.stride(1) != 1 or not t.is_cuda or t.dtype != out.dtype:
            raise KernelError(f"{nm} must be a CUDA matrix of {N} rows in {out.dtype} with unit column stride")
    if max(offsets[0], offsets[1]) + G * D > qkv.shape[1] or offsets[2] + H * Dv > qkv.shape[1]:
        raise KernelError(f"qkv of {qkv.shape[1]} columns does not hold the heads at {offsets}")
    if proj_offsets[0] + H * Dv > proj.shape[1] or max(proj_offsets[1], proj_offsets[2]) + H > proj.shape[1]:
        raise KernelError(f"proj of {proj.shape[1]} columns does not hold gate, b and a at {proj_offsets}")
    _want(A_log, "A_log", torch.float32, (H,))
    _want(dt_bias, "dt_bias", torch.float32, (H,))
    _want(norm_w, "norm_w", torch.float32, (Dv,))
    _want(state, "state", torch.float32)
    if state.shape[1:] != (H, D, Dv):
        raise KernelError(f"state must be [rows, {H}, {D}, {Dv}], got {tuple(state.shape)}")
    _want(seq_starts, "seq_starts", torch.int32, (R + 1,))
    _want(seq_rows, "seq_rows", torch.int32, (R,))
    if scratch is None:
        scratch = torch.empty(max(1, N * H * Dv), dtype=torch.float32, device=out.device)
    _want(scratch, "scratch", torch.float32)
    if scratch.numel() < N * H * Dv:
        raise KernelError(f"scratch of {scratch.numel()} elements for {N * H * Dv}")
    lib = library()
    check(lib, lib.sb_delta_rule(_ptr(out), _ptr(qkv), qkv.stride(0), offsets[0], offsets[1], offsets[2], _ptr(proj),
                                 proj.stride(0), proj_offsets[0], proj_offsets[1], proj_offsets[2], _ptr(A_log),
                                 _ptr(dt_bias), _ptr(norm_w), _ptr(state), _ptr(seq_starts), _ptr(seq_rows), R, H, G,
                                 D, Dv, float(eps), float(q_scale), _code(out.dtype), _ptr(scratch), N, _stream()),
          "delta_rule", kernels=2)


def moe_logits(logits: torch.Tensor, x: torch.Tensor, router: torch.Tensor) -> None:
    """logits float32 [N, E] = x [N, K] @ router [E, K]^T with float32 weights and sums; every token's sums are
    made in the same order whatever else the step holds."""
    N, K = x.shape
    E = router.shape[0]
    _want(x, "x")
    _want(router, "router", torch.float32, (E, K))
    _want(logits, "logits", torch.float32, (N, E))
    lib = library()
    check(lib, lib.sb_moe_logits(_ptr(logits), _ptr(x), _ptr(router), N, E, K, _code(x.dtype), _stream()), "moe_logits")


def moe_route(logits: torch.Tensor, correction: Optional[torch.Tensor], weights: torch.Tensor, ids: torch.Tensor,
              picked: torch.Tensor, groups: int, keep: int, top: int) -> None:
    """Choose `top` of E router outputs per token: s = softmax(logits); chosen by s + correction among the
    `keep` best of `groups` equal groups of neighbours (a group's score is its largest s + correction);
    weights float32 [N, E] gets s at the chosen outputs and 0 elsewhere, ids int32 / picked float32 [N, top]
    the choices best first."""
    N, E = logits.shape
    _want(logits, "logits", torch.float32)
    if correction is not None:
        _want(correction, "correction", torch.float32, (E,))
    _want(weights, "weights", torch.float32, (N, E))
    _want(ids, "ids", torch.int32, (N, top))
    _want(picked, "picked", torch.float32, (N, top))
    lib = library()
    check(lib, lib.sb_moe_route(_ptr(logits), _ptr(correction), _ptr(weights), _ptr(ids), _ptr(picked), N, E,
                                int(groups), int(keep), int(top), _stream()), "moe_route")


def moe_scale(act: torch.Tensor, weights: torch.Tensor, experts: int) -> None:
    """act[n, e*F + f] *= weights[n, e] for the `experts` first columns of weights; act [N, experts*F]."""
    N, width = act.shape
    _want(act, "act")
    _want(weights, "weights", torch.float32)
    if weights.shape[0] != N or weights.shape[1] < experts or width % experts:
        raise KernelError(f"weights {tuple(weights.shape)} do not fit activations {tuple(act.shape)} of {experts} experts")
    lib = library()
    check(lib, lib.sb_moe_scale(_ptr(act), _ptr(weights), N, weights.shape[1], int(experts), width // experts,
                                _code(act.dtype), _stream()), "moe_scale")


def moe_passthrough(slab: torch.Tensor, x: torch.Tensor, weights: torch.Tensor, first_identity: int) -> None:
    """slab[n, :] = x[n, :] * sum(weights[n, first_identity:]); slab float32 [N, d], x [N, d]."""
    N, d = x.shape
    _want(x, "x")
    _want(slab, "slab", torch.float32, (N, d))
    _want(weights, "weights", torch.float32)
    if weights.shape[0] != N:
        raise KernelError(f"weights {tuple(weights.shape)} for {N} tokens")
    lib = library()
    check(lib, lib.sb_moe_passthrough(_ptr(slab), _ptr(x), _ptr(weights), N, weights.shape[1], int(first_identity), d,
                                      _code(x.dtype), _stream()), "moe_passthrough")


def moe_table(weights: torch.Tensor, ids: torch.Tensor, table: torch.Tensor,
              feedback: Optional[torch.Tensor] = None) -> None:
    """Routing by a table: weights[n, e] = 1 / top if e is among table[ids[n], :], else 0.  weights float32
    [N, E]; ids int32 [N] (an id -1 - j stands for feedback[j], as in `embed`); table int32 [V, top]."""
    N, E = weights.shape
    _want(weights, "weights", torch.float32)
    _want(ids, "ids", torch.int32, (N,))
    _want(table, "table", torch.int32)
    if table.dim() != 2 or not 1 <= table.shape[1] <= E:
        raise KernelError(f"table must be [vocab, 1..{E}], got {tuple(table.shape)}")
    if feedback is not None:
        _want(feedback, "feedback", torch.int32)
    lib = library()
    check(lib, lib.sb_moe_table(_ptr(weights), _ptr(ids), _ptr(feedback), _ptr(table), N, E, table.shape[1],
                                table.shape[0], _stream()), "moe_table")


def softcap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place; x float32."""
    _want(x, "x", torch.float32)
    lib = library()
    check(lib, lib.sb_softcap(_ptr(x), x.numel(), float(cap), _stream()), "softcap")


# Differential attention: two score maps per head over one set of values.

def _diff_shapes(out, q, k_pool, v_pool, num_heads):
    N = q.shape[0]
    pages, Hkv, BS, Dk2 = k_pool.shape
    if Dk2 % 2:
        raise KernelError(f"key rows of {Dk2} dims do not hold two maps")
    dim, Dv = Dk2 // 2, v_pool.shape[3]
    _want(q, "q", k_pool.dtype, (N, num_heads * 2 * dim))
    _want(out, "out", q.dtype, (N, num_heads * Dv))
    _want(k_pool, "k_pool")
    _want(v_pool, "v_pool", k_pool.dtype, (pages, Hkv, BS, Dv))
    return N, Hkv, BS, dim, Dv


def attention_diff(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                   block_table: torch.Tensor, token_rows: torch.Tensor, positions: torch.Tensor, num_heads: int,
                   scale: float, lam: float, eps: float, out_scale: float, window: int = 0, keep_first: int = 0,
                   num_partitions: int = 1, part_o: Optional[torch.Tensor] = None,
                   part_ml: Optional[torch.Tensor] = None) -> None:
    """Paged causal differential attention, one query per token.  q [N, H*2*dim] holds per head [map 1 | map 2],
    k_pool [pages, Hkv, BS, 2*dim] likewise, v_pool [pages, Hkv, BS, Dv], out [N, H*Dv]:
    o = softmax(s1) v - lam * softmax(s2) v, then o / sqrt(mean(o^2) + eps) * out_scale per head.  Query i sees
    key j <= i if i - j < window or j < keep_first (window 0: every key).  All arithmetic is float32.
    With `num_partitions` > 1 the visible keys are cut into equal shares, one block each, merged by a second
    kernel through the float32 scratch part_o (N*H*2*NP*Dv) and part_ml (N*H*2*NP*2)."""
    N, Hkv, BS, dim, Dv = _diff_shapes(out, q, k_pool, v_pool, num_heads)
    _want(block_table, "block_table", torch.int32)
    _want(token_rows, "token_rows", torch.int32, (N,))
    _want(positions, "positions", torch.int32, (N,))
    if num_partitions > 1:
        _want(part_o, "part_o", torch.float32)
        _want(part_ml, "part_ml", torch.float32)
        if part_o.numel() < N * num_heads * 2 * num_partitions * Dv or part_ml.numel() < N * num_heads * 4 * num_partitions:
            raise KernelError("attention scratch buffers are too small")
    lib = library()
    check(lib, lib.sb_attention_diff(_ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                     block_table.shape[1], _ptr(token_rows), _ptr(positions), N, num_heads, Hkv, dim, Dv,
                                     BS, int(window), int(keep_first), float(scale), float(lam), float(eps),
                                     float(out_scale), int(num_partitions), _ptr(part_o), _ptr(part_ml), _code(q.dtype),
                                     _stream()), "attention_diff", kernels=2 if num_partitions > 1 else 1)


def attention_diff_tile_supports(num_heads: int, num_kv_heads: int, map_dim: int, value_dim: int,
                                 dtype: torch.dtype) -> bool:
    """Whether the tile kernel for prompt portions takes this shape (maps whose rows are whole 16-byte pieces,
    up to 128 dims; value heads up to 128 dims)."""
    return bool(library().sb_attention_diff_tile_supports(num_heads, num_kv_heads, map_dim, value_dim, _code(dtype)))


def attention_diff_tile(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                        block_table: torch.Tensor, seq_starts: torch.Tensor, seq_rows: torch.Tensor,
                        seq_first_pos: torch.Tensor, num_heads: int, scale: float, lam: float, eps: float,
                        out_scale: float, window: int = 0, keep_first: int = 0) -> None:
    """`attention_diff` for prompt portions: request r brings tokens seq_starts[r] .. seq_starts[r+1]-1 at
    positions seq_first_pos[r], +1, ... of cache row seq_rows[r]; a block serves a tile of consecutive tokens of
    one request.  The same arithmetic in float32."""
    N, Hkv, BS, dim, Dv = _diff_shapes(out, q, k_pool, v_pool, num_heads)
    R = seq_rows.numel()
    _want(block_table, "block_table", torch.int32)
    _want(seq_starts, "seq_starts", torch.int32, (R + 1,))
    _want(seq_rows, "seq_rows", torch.int32, (R,))
    _want(seq_first_pos, "seq_first_pos", torch.int32, (R,))
    lib = library()
    check(lib, lib.sb_attention_diff_tile(_ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                          block_table.shape[1], _ptr(seq_starts), _ptr(seq_rows), _ptr(seq_first_pos),
                                          R, N, num_heads, Hkv, dim, Dv, BS, int(window), int(keep_first), float(scale),
                                          float(lam), float(eps), float(out_scale), _code(q.dtype), _stream()),
          "attention_diff_tile")


def diff_combine(out: torch.Tensor, maps: torch.Tensor, num_heads: int, lam: float, eps: float, out_scale: float) -> None:
    """maps float32 [N, H*2*Dv] holds per head the outputs of its two maps, [a1 | a2]:
    out[n, h] = o / sqrt(mean(o^2) + eps) * out_scale with o = a1 - lam * a2; out [N, H*Dv] in the model dtype."""
    N = maps.shape[0]
    Dv = maps.shape[1] // (2 * num_heads)
    _want(maps, "maps", torch.float32, (N, num_heads * 2 * Dv))
    _want(out, "out", None, (N, num_heads * Dv))
    lib = library()
    check(lib, lib.sb_diff_combine(_ptr(out), _ptr(maps), N, num_heads, Dv, float(lam), float(eps), float(out_scale),
                                   _code(out.dtype), _stream()), "diff_combine")


# Residual streams (hyper-connections), gated recurrences, attention with mixed scores, latent attention's
# small steps.
def hyper_fold_norm(streams: torch.Tensor, init: Optional[torch.Tensor], branch_a: Optional[torch.Tensor],
                    scale_a: float, branch_b: Optional[torch.Tensor], scale_b: float, bias: Optional[torch.Tensor],
                    mix: Optional[torch.Tensor], out_weights: Optional[torch.Tensor], mult: float,
                    in_weights: Optional[torch.Tensor], gain: Optional[torch.Tensor], eps: float, center: bool,
                    out: Optional[torch.Tensor], row_index: Optional[torch.Tensor] = None,
                    read_out: Optional[torch.Tensor] = None) -> None:
    """One pass over rows of `s` residual streams, streams float32 [N, s, d] (s = 1: [N, d], the ordinary
    residual):
        y   = scale_a * (sum(branch_a, 0) + bias) + scale_b * sum(branch_b, 0)     (what a sublayer left; optional)
        x_t <- sum_f mix[f, t] x_f + mult * out_weights[t] * y                      (mix None: identity)
        u   = sum_t in_weights[t] x_t                                               (None: the plain sum)
        out = layer_norm(u) * gain (center) | rms_norm(u) * gain | u (gain None)
    `init` float32 [N, d]: the streams do not exist yet and all start as init.  With `row_index` only those
    rows are read and the streams stay as they are.  `read_out` float32 [M, d] receives u itself."""
    _want(streams, "streams", torch.float32)
    if streams.dim() == 2:
        N, d = streams.shape
        s = 1
    elif streams.dim() == 3:
        N, s, d = streams.shape
    else:
        raise KernelError(f"streams must be [N, s, d] or [N, d], got {tuple(streams.shape)}")
    if init is not None:
        _want(init, "init", torch.float32, (N, d))

    def parts(t, name):
        if t is None:
            return 0
        _want(t, name, torch.float32)
        if t.dim() != 3 or t.shape[1:] != (N, d):
            raise KernelError(f"{name} must be [S, {N}, {d}], got {tuple(t.shape)}")
        return t.shape[0]

    SA, SB = parts(branch_a, "branch_a"), parts(branch_b, "branch_b")
    for t, name, shape in ((bias, "bias", (d,)), (mix, "mix", (s, s)), (out_weights, "out_weights", (s,)),
                           (in_weights, "in_weights", (s,)), (gain, "gain", (d,))):
        if t is not None:
            _want(t, name, torch.float32, shape)
    M = N
    if row_index is not None:
        _want(row_index, "row_index", torch.int32)
        M = row_index.numel()
    if out is not None:
        _want(out, "out", None, (M, d))
    if read_out is not None:
        _want(read_out, "read_out", torch.float32, (M, d))
    lib = library()
    check(lib, lib.sb_hyper_fold_norm(_ptr(streams), _ptr(init), s, d, _ptr(branch_a), SA, N * d, float(scale_a),
                                      _ptr(branch_b), SB, N * d, float(scale_b), _ptr(bias), _ptr(mix),
                                      _ptr(out_weights), float(mult), _ptr(in_weights), _ptr(gain), float(eps),
                                      int(bool(center)), _ptr(out), _ptr(read_out), _ptr(row_index), M,
                                      _code(out.dtype) if out is not None else 0, _stream()), "hyper_fold_norm")


def min_gru(out: torch.Tensor, proj: torch.Tensor, bias_z: Optional[torch.Tensor], bias_x: Optional[torch.Tensor],
            state: torch.Tensor, seq_starts: torch.Tensor, seq_rows: torch.Tensor, longest: Optional[int] = None) -> None:
    """z = sigmoid(proj[:, :W] + bias_z); u = proj[:, W:2W] + bias_x; c = u + 1/2 where u >= 0, sigmoid(u) below;
    S <- (1 - z) S + z c per channel, token after token of every request; out = S * silu(proj[:, 2W:3W]).
    proj [N, >= 3W] in out's dtype; state float32 [rows, W] (the request's slot, carried on); out [N, W].
    `longest`: an upper bound of the tokens one request brings (default N - R + 1); long portions are cut into
    segments that run side by side and are joined in order."""
    N, W = out.shape
    _want(out, "out")
    if proj.dim() != 2 or proj.shape[0] != N or proj.shape[1] < 3 * W or proj.stride(1) != 1 or proj.dtype != out.dtype:
        raise KernelError(f"proj must be [{N}, >= {3 * W}] in {out.dtype} with unit column stride")
    _want(state, "state", torch.float32)
    if state.dim() != 2 or state.shape[1] != W:
        raise KernelError(f"state must be [rows, {W}], got {tuple(state.shape)}")
    for b, nm in ((bias_z, "bias_z"), (bias_x, "bias_x")):
        if b is not None:
            _want(b, nm, torch.float32, (W,))
    R = seq_rows.numel()
    _want(seq_starts, "seq_starts", torch.int32, (R + 1,))
    _want(seq_rows, "seq_rows", torch.int32, (R,))
    lib = library()
    check(lib, lib.sb_min_gru(_ptr(out), _ptr(proj), proj.stride(0), _ptr(bias_z), _ptr(bias_x), _ptr(state),
                              _ptr(seq_starts), _ptr(seq_rows), R, W, int(longest if longest is not None else N - R + 1),
                              _code(out.dtype), _stream()), "min_gru")


def gated_linear_attention_supports(key_dim: int, value_dim: int) -> bool:
    return bool(library().sb_gated_linear_attention_supports(key_dim, value_dim))


def gated_linear_attention(out: torch.Tensor, proj: torch.Tensor, offsets: Tuple[int, int, int],
                           f_bias: Optional[torch.Tensor], lower: Optional[torch.Tensor], norm_w: torch.Tensor,
                           state: torch.Tensor, seq_starts: torch.Tensor, seq_rows: torch.Tensor, num_heads: int,
                           key_dim: int, value_dim: int, eps: float, scratch: torch.Tensor,
                           longest: Optional[int] = None, seg_scratch: Optional[torch.Tensor] = None) -> None:
    """Linear attention whose forget gate also decides what is written, token after token of every request:
    q = silu(proj_q); f = lower + (1 - lower) * sigmoid(proj_f + f_bias); S <- diag(f) S + (1 - f) v^T; o = S^T q;
    out = o / sqrt(mean(o^2) + eps) * norm_w per head.  `offsets` = columns where q (H*D), f (H*D) and v (H*Dv)
    begin in proj; state float32 [rows, H, D, Dv]; scratch float32 [N, H*Dv] (the raw o).
    `longest`: an upper bound of the tokens one request brings (default N - R + 1).  Long portions are cut into
    `gated_linear_attention_segments(longest)` segments that run side by side and are joined in order; with more
    than one, `seg_scratch` float32 of `gated_linear_attention_seg_scratch(R, longest, H, D, Dv)` values is needed."""
    H, D, Dv = num_heads, key_dim, value_dim
    N = out.shape[0]
    _want(out, "out", None, (N, H * Dv))
    if proj.dim() != 2 or proj.shape[0] != N or proj.stride(1) != 1 or proj.dtype != out.dtype:
        raise KernelError(f"proj must be [{N}, columns] in {out.dtype} with unit column stride")
    q_off, f_off, v_off = offsets
    if max(q_off + H * D, f_off + H * D, v_off + H * Dv) > proj.shape[1]:
        raise KernelError("the column offsets reach past the rows of proj")
    _want(state, "state", torch.float32)
    if state.dim() != 4 or state.shape[1:] != (H, D, Dv):
        raise KernelError(f"state must be [rows, {H}, {D}, {Dv}], got {tuple(state.shape)}")
    for t, nm in ((f_bias, "f_bias"), (lower, "lower")):
        if t is not None:
            _want(t, nm, torch.float32, (H * D,))
    _want(norm_w, "norm_w", torch.float32, (Dv,))
    _want(scratch, "scratch", torch.float32)
    if scratch.numel() < N * H * Dv:
        raise KernelError("the scratch buffer is too small")
    R = seq_rows.numel()
    _want(seq_starts, "seq_starts", torch.int32, (R + 1,))
    _want(seq_rows, "seq_rows", torch.int32, (R,))
    longest = N - R + 1 if longest is None else int(longest)
    segs = gated_linear_attention_segments(longest)
    if segs > 1:
        if seg_scratch is None:
            raise KernelError(f"{segs} segments need seg_scratch")
        _want(seg_scratch, "seg_scratch", torch.float32)
        if seg_scratch.numel() < gated_linear_attention_seg_scratch(R, longest, H, D, Dv):
            raise KernelError("seg_scratch is too small")
    lib = library()
    check(lib, lib.sb_gated_linear_attention(_ptr(out), _ptr(proj), proj.stride(0), q_off, f_off, v_off, _ptr(f_bias),
                                             _ptr(lower), _ptr(norm_w), _ptr(state), _ptr(seq_starts), _ptr(seq_rows),
                                             R, H, D, Dv, float(eps), _code(out.dtype), _ptr(scratch), N, segs,
                                             _ptr(seg_scratch) if segs > 1 else None, _stream()),
          "gated_linear_attention", kernels=3 if segs > 1 else 2)


def gated_linear_attention_segments(longest: int) -> int:
    return int(library().sb_gated_linear_attention_segments(int(longest)))


def gated_linear_attention_seg_scratch(R: int, longest: int, H: int, D: int, Dv: int) -> int:
    """float32 values of scratch the segments of `gated_linear_attention` need (0 with one segment)."""
    segs = gated_linear_attention_segments(longest)
    return 0 if segs == 1 else R * (segs + 1) * H * D * (Dv + 1)


def glu_clamp(out: torch.Tensor, x: torch.Tensor, bias_gate: Optional[torch.Tensor], bias_up: Optional[torch.Tensor],
              limit: float, alpha: float, offset: float) -> None:
    """g = min(x[:, :F] + bias_gate, limit); u = clamp(x[:, F:] + bias_up, -limit, limit);
    out = g * sigmoid(alpha * g) * (u + offset).  x [N, 2F] in out's dtype or float32 partial sums [S, N, 2F]."""
    N, F_ = out.shape
    _want(out, "out")
    parts = x.dim() == 3
    if parts:
        _want(x, "x partial sums", torch.float32, (x.shape[0], N, 2 * F_))
    else:
        _want(x, "x", out.dtype, (N, 2 * F_))
    for b, nm in ((bias_gate, "bias_gate"), (bias_up, "bias_up")):
        if b is not None:
            _want(b, nm, torch.float32, (F_,))
    lib = library()
    check(lib, lib.sb_glu_clamp(_ptr(out), None if parts else _ptr(x), _ptr(x) if parts else None,
                                x.shape[0] if parts else 0, N * 2 * F_, _ptr(bias_gate), _ptr(bias_up), N, F_,
                                float(limit), float(alpha), float(offset), _code(out.dtype), _stream()), "glu_clamp")


def scale_(x: torch.Tensor, c: float) -> None:
    """x *= c in place; x float32."""
    _want(x, "x", torch.float32)
    lib = library()
    check(lib, lib.sb_scale(_ptr(x), x.numel(), float(c), _stream()), "scale")


def segment_norm(x: torch.Tensor, segments, eps: float) -> None:
    """Runs of columns of x [N, columns], each RMS-normed over its own length with a gain (None: copied as it
    is) and written to one or two places.  `segments`: up to four (begin, length, gain, [(tensor, column), ...])
    with one or two destinations, matrices [N, >= column + length] of x's dtype with unit column stride."""
    if x.dim() != 2 or x.stride(1) != 1 or not x.is_cuda:
        raise KernelError("x must be a CUDA matrix with unit column stride")
    N, n = x.shape[0], len(segments)
    if not 1 <= n <= 4:
        raise KernelError("segment_norm takes one to four segments")
    IntArr, PtrArr, LLArr = ctypes.c_int * n, ctypes.c_void_p * n, ctypes.c_longlong * n
    begin, length, gains = IntArr(), IntArr(), PtrArr()
    d0, s0, o0, d1, s1, o1 = PtrArr(), LLArr(), IntArr(), PtrArr(), LLArr(), IntArr()
    for i, (b, ln, gain, places) in enumerate(segments):
        if b < 0 or ln < 1 or b + ln > x.shape[1]:
            raise KernelError(f"segment {i} ({b}, {ln}) lies outside the {x.shape[1]} columns")
        if gain is not None:
            _want(gain, "gain", torch.float32, (ln,))
        if not 1 <= len(places) <= 2:
            raise KernelError("a segment goes to one or two places")
        begin[i], length[i], gains[i] = b, ln, _ptr(gain)
        for j, (t, col) in enumerate(places):
            if (t.dim() != 2 or t.shape[0] != N or t.stride(1) != 1 or t.dtype != x.dtype or col < 0
                    or col + ln > t.shape[1]):
                raise KernelError(f"a destination must be [{N}, >= {col + ln}] in {x.dtype} with unit column stride")
            if j == 0:
                d0[i], s0[i], o0[i] = t.data_ptr(), t.stride(0), col
            else:
                d1[i], s1[i], o1[i] = t.data_ptr(), t.stride(0), col
        if len(places) == 1:
            d1[i], s1[i], o1[i] = None, 0, 0
    lib = library()
    check(lib, lib.sb_segment_norm(_ptr(x), x.stride(0), n, begin, length, gains, d0, s0, o0, d1, s1, o1, float(eps), N,
                                   _code(x.dtype), _stream()), "segment_norm")


def head_matmul(y: torch.Tensor, y_off: int, y_head: int, x: torch.Tensor, x_off: int, x_head: int, w: torch.Tensor,
                num_heads: int, transposed: bool, carry: int = 0) -> None:
    """A matrix per head: with W_h = rows h*A .. h*A + A - 1 of w [H*A, B],
    y[n, y_off + h*y_head + :] = W_h x[n, x_off + h*x_head + :B]  (A outputs), or, `transposed`,
    W_h^T x[n, x_off + h*x_head + :A]  (B outputs).  `carry`: the values in front of every head's input are
    copied in front of its output.  Sums are float32; x, y, w share one dtype."""
    H = num_heads
    if w.dim() != 2 or w.shape[0] % H:
        raise KernelError(f"w must be [{H} * A, B], got {tuple(w.shape)}")
    A, B = w.shape[0] // H, w.shape[1]
    _want(w, "w", x.dtype)
    nin, nout = (A, B) if transposed else (B, A)
    N = x.shape[0]
    for t, nm, off, head, n in ((x, "x", x_off, x_head, nin), (y, "y", y_off, y_head, nout)):
        if t.dim() != 2 or t.shape[0] != N or t.stride(1) != 1 or t.dtype != x.dtype or not t.is_cuda:
            raise KernelError(f"{nm} must be a CUDA matrix [{N}, columns] in {x.dtype} with unit column stride")
        if off + (H - 1) * head + n > t.shape[1] or off < carry:
            raise KernelError(f"{nm}: {H} heads of {n} at {off} + h * {head} do not fit {t.shape[1]} columns")
    lib = library()
    check(lib, lib.sb_head_matmul(_ptr(y), y.stride(0), y_off, y_head, _ptr(x), x.stride(0), x_off, x_head, _ptr(w),
                                  H, A, B, int(bool(transposed)), int(carry), N, _code(x.dtype), _stream()),
          "head_matmul")


def latent_write(down: torch.Tensor, c_off: int, r_off: int, rank: int, rot_dim: int, gain: torch.Tensor, eps: float,
                 q: torch.Tensor, num_heads: int, inv_freq: torch.Tensor, neighbours: bool, magnitude: float,
                 positions: torch.Tensor, token_rows: torch.Tensor, block_table: torch.Tensor, k_pool: torch.Tensor,
                 v_pool: torch.Tensor) -> None:
    """Per token: c = rmsnorm(down[:, c_off : c_off + rank]) * gain; the key part down[:, r_off : r_off + rot_dim]
    and the first rot_dim dims of every head of q [N, H * (rot_dim + rank)] are turned by the token's position
    (q in place); the row [turned key part | c] is written to the token's slot of k_pool [pages, 1, BS, rot_dim +
    rank] and c to v_pool [pages, 1, BS, rank].  Norm and angles are float32."""
    N, D = q.shape[0], rot_dim + rank
    _want(q, "q", None, (N, num_heads * D))
    if down.dim() != 2 or down.shape[0] != N or down.stride(1) != 1 or down.dtype != q.dtype or not down.is_cuda:
        raise KernelError(f"down must be a CUDA matrix [{N}, columns] in {q.dtype} with unit column stride")
    if max(c_off + rank, r_off + rot_dim) > down.shape[1]:
        raise KernelError("the column offsets reach past the rows of down")
    _want(gain, "gain", torch.float32, (rank,))
    _want(inv_freq, "inv_freq", torch.float32)
    if inv_freq.numel() < rot_dim // 2:
        raise KernelError(f"inv_freq has {inv_freq.numel()} entries for {rot_dim} turning dims")
    _want(positions, "positions", torch.int32, (N,))
    _want(token_rows, "token_rows", torch.int32, (N,))
    _want(block_table, "block_table", torch.int32)
    _want(k_pool, "k_pool", q.dtype)
    if k_pool.dim() != 4 or k_pool.shape[1] != 1 or k_pool.shape[3] != D:
        raise KernelError(f"k_pool must be [pages, 1, page_size, {D}], got {tuple(k_pool.shape)}")
    _want(v_pool, "v_pool", q.dtype, (*k_pool.shape[:3], rank))
    lib = library()
    check(lib, lib.sb_latent_write(_ptr(down), down.stride(0), c_off, r_off, rank, rot_dim, _ptr(gain), float(eps),
                                   _ptr(q), num_heads, _ptr(inv_freq), int(bool(neighbours)), float(magnitude),
                                   _ptr(positions), _ptr(token_rows), _ptr(block_table), block_table.shape[1],
                                   k_pool.shape[2], _ptr(k_pool), _ptr(v_pool), N, _code(q.dtype), _stream()),
          "latent_write")


def attention_talk_tile(num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int) -> int:
    """Queries per tile the mixed-score attention kernel chooses for prompt portions; 0: it does not take the shape."""
    return int(library().sb_attention_talk_tile(num_heads, num_kv_heads, key_dim, value_dim))


def attention_talk(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                   block_table: torch.Tensor, seq_starts: torch.Tensor, seq_rows: torch.Tensor,
                   seq_first_pos: torch.Tensor, talk: torch.Tensor, num_heads: int, scale: float, window: int = 0,
                   gate: Optional[torch.Tensor] = None, queries_per_tile: int = 0, num_partitions: int = 1,
                   part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None) -> None:
    """Paged causal attention whose scaled scores are mixed across heads before the softmax:
    s_h = scale * sum_g talk[h, g] (q_g . k_kv(g)); o_h = softmax(s_h) v_kv(h) * sigmoid(gate_h) (gate [N, >= Hq*Dv],
    optional).  Request r brings tokens seq_starts[r] .. seq_starts[r+1]-1 at positions seq_first_pos[r], +1, ...
    of cache row seq_rows[r].  q [N, Hq*Dk], pools [pages, Hkv, BS, Dk | Dv], out [N, Hq*Dv].
    `queries_per_tile` 0: chosen from the shape; 1 with `num_partitions` > 1 for decode steps: every token's keys
    are cut into shares merged through float32 scratch part_o (N*Hq*NP*Dv) and part_ml (N*Hq*NP*2)."""
    N = q.shape[0]
    pages, Hkv, BS, Dk = k_pool.shape
    Dv = v_pool.shape[3]
    Hq = num_heads
    R = seq_rows.numel()
    _want(q, "q", k_pool.dtype, (N, Hq * Dk))
    _want(out, "out", q.dtype, (N, Hq * Dv))
    _want(k_pool, "k_pool")
    _want(v_pool, "v_pool", k_pool.dtype, (pages, Hkv, BS, Dv))
    _want(block_table, "block_table", torch.int32)
    _want(seq_starts, "seq_starts", torch.int32, (R + 1,))
    _want(seq_rows, "seq_rows", torch.int32, (R,))
    _want(seq_first_pos, "seq_first_pos", torch.int32, (R,))
    _want(talk, "talk", torch.float32, (Hq, Hq))
    gate_stride = _gate_stride(gate, q, N, Hq * Dv)
    if num_partitions > 1:
        _want(part_o, "part_o", torch.float32)
        _want(part_ml, "part_ml", torch.float32)
        if part_o.numel() < N * Hq * num_partitions * Dv or part_ml.numel() < N * Hq * num_partitions * 2:
            raise KernelError("attention scratch buffers are too small")
    lib = library()
    check(lib, lib.sb_attention_talk(_ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                     block_table.shape[1], _ptr(seq_starts), _ptr(seq_rows), _ptr(seq_first_pos), R,
                                     _ptr(talk), _ptr(gate), gate_stride, N, Hq, Hkv, Dk, Dv, BS, int(window),
                                     float(scale), int(queries_per_tile), int(num_partitions), _ptr(part_o),
                                     _ptr(part_ml), _code(q.dtype), _stream()), "attention_talk",
          kernels=2 if num_partitions > 1 else 1)


def attention_talk_dense_step(step: int, q, k_pool, v_pool, table_row, Kc, Vt, Qg, S, P, O, out, gate, talk,
                              num_heads: int, C: int, Cp: int, n0: int, nb: int, pos0: int, window: int, scale: float) -> None:
    """One of the steps between the matrix products of the tensor-core form of `attention_talk` for one long prompt
    portion (bfloat16): 0 gathers the request's C keys and values out of their pages (Kc [Hkv, Cp, Dk]; Vt [Hkv, Dv,
    2*Cp], the transposed values twice side by side); 1 gathers the queries n0 .. n0+nb-1 (Qg [Hkv, G*nb, Dk]); 2
    mixes the raw scores S [Hkv, G*nb, Cp] across the heads, masks, takes the softmax in float32 and writes P [Hkv,
    G*nb, 2*Cp], every weight as a high and a low bfloat16 term; 3 writes O [Hkv, G*nb, Dv] to out [N, H*Dv], gated."""
    pages, Hkv, BS, Dk = k_pool.shape
    Dv = v_pool.shape[3]
    for t in (q, k_pool, v_pool, Kc, Vt, Qg, P, out):
        _want(t, "a matrix of the dense form", torch.bfloat16)
    for t in (S, O, talk):
        _want(t, "a float32 matrix of the dense form", torch.float32)
    _want(table_row, "table_row", torch.int32)
    G = num_heads // Hkv
    if (Kc.numel() < Hkv * Cp * Dk or Vt.numel() < Hkv * Dv * 2 * Cp or Qg.numel() < num_heads * nb * Dk
            or S.numel() < num_heads * nb * Cp or P.numel() < num_heads * nb * 2 * Cp or O.numel() < num_heads * nb * Dv):
        raise KernelError("a matrix of the dense form is too small")
    gate_stride = _gate_stride(gate, q, q.shape[0], num_heads * Dv)
    lib = library()
    check(lib, lib.sb_attention_talk_dense(int(step), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(table_row), _ptr(Kc),
                                           _ptr(Vt), _ptr(Qg), _ptr(S), _ptr(P), _ptr(O), _ptr(out), _ptr(gate),
                                           gate_stride, _ptr(talk), num_heads, Hkv, Dk, Dv, BS, int(C), int(Cp), int(n0),
                                           int(nb), int(pos0), int(window), float(scale), _stream()),
          "attention_talk_dense")
