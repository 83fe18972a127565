"""Python faces of the CUDA kernels: they check their arguments and launch on torch's current stream.

Every function here runs a hand-written kernel from csrc/; none has a CPU or
library fallback. Tensors must live on the GPU and be contiguous where a kernel
assumes it; a kernel that does not take a size raises KernelRefused with the
reason instead of computing something else.
"""
import ctypes

import torch

from . import guards
from .build import load_module

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


class KernelRefused(KernelError):
    """The sizes or types given are outside what the kernel is built for."""


def _dt(t):
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {t.dtype} is neither float32 nor bfloat16")


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream():
    # torch's current stream as a raw handle (the public torch.cuda.current_stream() builds a Stream object
    # for it and takes fifty times as long: a few microseconds on every launch)
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("a kernel was given a tensor that is not on the GPU; there is no CPU path")


LAUNCHES = 0  # kernels launched through this module (a captured graph's replays are not counted here)


def _check(lib, rc, what, kernels=1):
    global LAUNCHES
    if rc == 0:
        LAUNCHES += kernels
        return
    if rc < 0:
        raise KernelRefused(lib.abk_last_error().decode())
    raise KernelError(f"{what}: CUDA error {rc} at launch")


_i, _ll, _f = ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def fill_normal(out, key, mean, amplitude, first=0):
    """out.flat[i] = mean + amplitude * z(key, first + i), z a unit normal that depends on (key, index) alone
    (csrc/utility.cu; weights/random_init.py holds the host twin). out float32 or bfloat16, contiguous."""
    _need_cuda(out)
    lib = load_module("utility")
    assert out.is_contiguous()
    _check(lib, lib.abk_fill_normal(_p(out), _i(_dt(out)), _ll(out.numel()), _ll(first), ctypes.c_ulonglong(key),
                                    _f(mean), _f(amplitude), _stream()), "fill_normal")


def embed(tokens, table, x, status):
    """x[t] = float(table[tokens[t]]) (src/model.c:290-291). tokens int32 [T], x float32 [T, d]."""
    _need_cuda(tokens, table, x, status)
    lib = load_module("elementwise")
    n, d = x.shape
    assert tokens.dtype == torch.int32 and x.dtype == torch.float32 and tokens.numel() >= n
    assert table.is_contiguous() and x.is_contiguous() and table.shape[1] == d
    _check(lib, lib.abk_embed(_p(tokens), _p(table), _i(_dt(table)), _p(x), _i(n), _i(d), _i(table.shape[0]),
                              _p(status), _stream()), "embed")


def add_rmsnorm(x, y, weight, out, eps, rows=None, n_rows=None):
    """x += y (if given); out = weight * x / sqrt(mean(x^2) + eps) (src/model.c:238-244).

    rows (int32) picks the rows of x that are normed into out[0:len(rows)]; x is then left unchanged.
    """
    _need_cuda(x, y, weight, out, rows)
    lib = load_module("elementwise")
    d = x.shape[-1]
    n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == d
    assert y is None or (y.dtype == torch.float32 and y.shape == x.shape and y.is_contiguous())
    assert x.is_contiguous() and out.is_contiguous() and out.shape[-1] == d and out.shape[0] >= n
    _check(lib, lib.abk_add_rmsnorm(_p(x), _p(y), _p(weight), _p(out), _i(_dt(out)), _p(rows), _i(n), _i(d),
                                    _f(eps), _stream()), "add_rmsnorm")


def swiglu(gate_up, act, block=None):
    """act = silu(gate) * up (src/model.c:274-282). A row of gate_up holds gate and up in turns of `block`
    columns (gate of features [0, block), up of the same, gate of the next block, ...); by default all gates
    and then all ups."""
    _need_cuda(gate_up, act)
    lib = load_module("elementwise")
    n, two_i = gate_up.shape
    assert act.shape == (n, two_i // 2) and act.dtype == gate_up.dtype
    assert gate_up.is_contiguous() and act.is_contiguous()
    _check(lib, lib.abk_swiglu(_p(gate_up), _p(act), _i(_dt(act)), _i(n), _i(two_i // 2), _i(block or two_i // 2),
                               _stream()), "swiglu")


def qkv_prep(qkv, n_heads, n_kv_heads, head_dim, batch, q_norm, k_norm, eps, cos, sin, rotary_dim, interleaved,
             cache, q_only=False, v_dim=None, row=None):
    """Per-head norm of q and k, rotary encoding, and the cache write of k and v (src/model.c:247-259).

    qkv [T, (Hq + 2 Hkv) * hd] is changed in place. batch: engine.batch.StepBatch. cache: a
    cache.LayerKV or None (nothing written). q_only: only the q heads are prepared.
    """
    _need_cuda(qkv, q_norm, k_norm, cos, sin)
    lib = load_module("elementwise")
    n = batch.n_rows
    vd = v_dim or head_dim
    heads_size = (n_heads + n_kv_heads) * head_dim + n_kv_heads * vd
    row = row or heads_size  # a row may have padding behind its heads
    assert qkv.is_contiguous() and qkv.shape[1] == row >= heads_size and qkv.shape[0] >= n
    if cos is not None:
        assert cos.dtype == torch.float32 and cos.shape == sin.shape and cos.shape[1] == rotary_dim // 2
        if batch.max_position >= cos.shape[0]:
            raise KernelError(f"position {batch.max_position} is beyond the rotary table of {cos.shape[0]} positions")
    if cache is not None:
        assert cache.k.dtype == qkv.dtype and cache.k.shape[1:] == (n_kv_heads, cache.tokens_per_page, head_dim)
        assert cache.v.shape[1:] == (n_kv_heads, cache.tokens_per_page, vd)
    pinned = cache.pinned_pages if cache is not None else 0
    if vd != head_dim or pinned or row != heads_size:  # the general kernel alone takes values of another size,
        # pinned first pages and padded rows
        _check(lib, lib.abk_qkv_prep_general(
            _p(qkv), _i(_dt(qkv)), _i(n), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(1 if q_only else 0),
            _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(batch.seq_len_after), _p(q_norm),
            _p(k_norm), _f(eps or 0.0), _p(cos), _p(sin), _i(rotary_dim), _i(1 if interleaved else 0),
            _p(cache.k if cache is not None else None), _p(cache.v if cache is not None else None),
            _p(cache.page_table if cache is not None else None), _i(cache.table_width if cache is not None else 0),
            _i(cache.ring_pages if cache is not None else 0), _i(cache.tokens_per_page if cache is not None else 1),
            _i(vd), _i(pinned), _ll(row), _stream()), "qkv_prep")
        return
    _check(lib, lib.abk_qkv_prep(
        _p(qkv), _i(_dt(qkv)), _i(n), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(1 if q_only else 0),
        _p(batch.token_seq),
        _p(batch.token_pos), _p(batch.seq_slot), _p(batch.seq_len_after), _p(q_norm), _p(k_norm), _f(eps or 0.0),
        _p(cos), _p(sin), _i(rotary_dim), _i(1 if interleaved else 0),
        _p(cache.k if cache is not None else None), _p(cache.v if cache is not None else None),
        _p(cache.page_table if cache is not None else None), _i(cache.table_width if cache is not None else 0),
        _i(cache.ring_pages if cache is not None else 0), _i(cache.tokens_per_page if cache is not None else 1),
        _stream()), "qkv_prep")


def advance_decode(batch):
    """Every row of a decode step one position on, on the device (engine.batch.StepBatch.advance_on_device)."""
    lib = load_module("elementwise")
    _check(lib, lib.abk_advance_decode(_p(batch.token_seq), _p(batch.token_pos), _i(batch.n_rows), _p(batch.seq_pos0),
                                       _p(batch.seq_len_after), _i(batch.n_seqs), _stream()), "advance_decode")


def attention_generic(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, from_step=False, v_dim=None,
                      keep_first=0, sink=None, exact_weights=False, row=None, chunk=None, softcap=None):
    """Causal grouped-query attention of every token of the step (src/model.c:197-211).

    q is read from qkv's q columns. Keys and values come from `cache` (a cache.LayerView), or, with
    from_step, from this step's own rows of qkv (only right when every sequence starts at position 0).
    v_dim: the size of a value head (default head_dim). keep_first (with a window): the sequence's first keys
    stay visible. sink: float32 [n_heads], a score per head that joins the denominator. exact_weights: the
    softmax's weights stay float32 in the second product. row: elements between rows of qkv where a row has padding
    behind its heads. chunk: a token sees only the keys of its own run of `chunk` positions (counted from the
    sequence's first). softcap: scores become softcap * tanh(score / softcap) after the scale.
    """
    _need_cuda(qkv, out, sink)
    lib = load_module("attention_generic")
    n = batch.n_rows
    vd = v_dim or head_dim
    heads_size = (n_heads + n_kv_heads) * head_dim + n_kv_heads * vd
    row = row or heads_size
    assert qkv.is_contiguous() and qkv.shape[1] == row >= heads_size and out.is_contiguous() and out.dtype == qkv.dtype
    assert out.shape[1] == n_heads * vd and out.shape[0] >= n and qkv.shape[0] >= n
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == n_heads)
    esize = qkv.element_size()
    k_step = ctypes.c_void_p(qkv.data_ptr() + n_heads * head_dim * esize) if from_step else ctypes.c_void_p(0)
    v_step = ctypes.c_void_p(qkv.data_ptr() + (n_heads + n_kv_heads) * head_dim * esize) if from_step else ctypes.c_void_p(0)
    if not from_step:
        assert cache is not None and cache.k.dtype == qkv.dtype and cache.v.shape[-1] == vd
    _check(lib, lib.abk_attention_chunked(
        _p(qkv), _ll(row), _p(out), _i(_dt(qkv)), _i(n), _i(n_heads), _i(n_kv_heads), _i(head_dim), _f(scale),
        _i(window or 0), _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(batch.seq_start),
        _p(batch.seq_pos0), _p(cache.k if cache is not None else None), _p(cache.v if cache is not None else None),
        _p(cache.page_table if cache is not None else None), _i(cache.table_width if cache is not None else 0),
        _i(cache.ring_pages if cache is not None else 0), _i(cache.tokens_per_page if cache is not None else 1),
        k_step, v_step, _ll(row), _i(vd), _i(keep_first or 0), _i(cache.pinned_pages if cache is not None else 0),
        _p(sink), _i(1 if exact_weights else 0), _i(chunk or 0), _f(softcap or 0.0), _stream()), "attention")


def gemm_simt(x, w, out, m=None):
    """out[:m] = x[:m] . w^T on the CUDA cores in float32, any sizes (src/model.c:299 and the like)."""
    _need_cuda(x, w, out)
    lib = load_module("gemm_simt")
    m = x.shape[0] if m is None else m
    n, k = w.shape
    assert x.shape[1] == k and out.shape[1] == n and x.shape[0] >= m and out.shape[0] >= m
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(lib, lib.abk_gemm_simt(_p(x), _i(_dt(x)), _p(w), _i(_dt(w)), _p(out), _i(_dt(out)), _i(m), _i(n), _i(k),
                                  _ll(x.stride(0)), _ll(w.stride(0)), _ll(out.stride(0)), _stream()), "gemm_simt")


def gemm_rows_takes(x, w, out, m):
    """Whether the weight-streaming kernel for a handful of rows takes this product."""
    k = w.shape[1]
    return (m <= 64 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 32 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1)


def gemm_rows(x, w, out, m=None):
    """out[:m] = x[:m] . w^T for m <= 16 rows: the weights stream once through warp-level tensor-core
    products, no scratch memory (src/model.c:299 and the like)."""
    _need_cuda(x, w, out)
    lib = load_module("gemm_rows")
    m = x.shape[0] if m is None else m
    n, k = w.shape
    assert x.shape[1] == k and out.shape[1] == n and x.shape[0] >= m and out.shape[0] >= m
    _check(lib, lib.abk_gemm_rows(_p(x), _p(w), _p(out), _i(_dt(out)), _i(m), _i(n), _i(k), _ll(x.stride(0)),
                                  _ll(w.stride(0)), _ll(out.stride(0)), _stream()), "gemm_rows")


def gemm_rows_planes(x, w, out, block, m=None, tanh_from=None):
    """Several products of a handful of rows in one launch: out[:m, i * block : (i + 1) * block] =
    x[i, :m] . w[i * block : (i + 1) * block]^T for every run i of `block` rows of w (the last run may be shorter).
    x [runs, rows, K] bfloat16 contiguous, w [N, K] bfloat16, out [rows, N] bfloat16 or float32; block a multiple of 16.
    tanh_from: output features from there on are tanh of their sums."""
    _need_cuda(x, w, out)
    lib = load_module("gemm_rows")
    runs, rows, k = x.shape
    m = rows if m is None else m
    n = w.shape[0]
    assert x.is_contiguous() and w.shape[1] == k and out.shape[1] == n and out.shape[0] >= m and -(-n // block) <= runs
    assert x.dtype == w.dtype == torch.bfloat16 and w.stride(1) == 1 and out.stride(1) == 1
    _check(lib, lib.abk_gemm_rows_planes(_p(x), _p(w), _p(out), _i(_dt(out)), _i(m), _i(n), _i(k), _ll(x.stride(1)),
                                         _ll(w.stride(0)), _ll(out.stride(0)), _i(block), _ll(x.stride(0)),
                                         _i(-1 if tanh_from is None else tanh_from), _stream()),
           "gemm_rows_planes")


def gemm_rows_swiglu(x, w_gate_up, act, m=None, block=None):
    """act[:m] = silu(x . gate^T) * (x . up^T) for m <= 64 rows, w_gate_up [2 I, K] holding gate and up rows in
    turns of `block` rows (by default all gates, then all ups): the feed-forward's first product and its
    activation in one kernel (src/model.c:307-308)."""
    _need_cuda(x, w_gate_up, act)
    lib = load_module("gemm_rows")
    m = x.shape[0] if m is None else m
    two_i, k = w_gate_up.shape
    assert x.shape[1] == k and act.shape[1] == two_i // 2 and act.dtype == torch.bfloat16 and act.stride(1) == 1
    _check(lib, lib.abk_gemm_rows_swiglu(_p(x), _p(w_gate_up), _p(act), _i(m), _i(two_i // 2), _i(k), _ll(x.stride(0)),
                                         _ll(w_gate_up.stride(0)), _ll(act.stride(0)), _i(block or two_i // 2), _stream()),
           "gemm_rows_swiglu")


def gemm_tc_swiglu_takes(x, w_gate_up, act, m, block):
    """Whether the tensor-core product with the activation in its epilogue takes this: many rows, gate and up
    rows in turns of 128."""
    return (block == 128 and m > 256 and act.dtype == torch.bfloat16 and w_gate_up.shape[0] % 256 == 0
            and act.stride(0) % 8 == 0 and act.data_ptr() % 16 == 0 and gemm_tc_takes(x, w_gate_up, act))


def gemm_tc_swiglu(x, w_gate_up, act, m=None):
    """act[:m] = silu(x . gate^T) * (x . up^T) on the tcgen05 tensor cores for more than 256 rows, w_gate_up
    [2 I, K] holding gate and up rows in turns of 128: the activation runs in the product's epilogue, under the
    next tile's multiplication (src/model.c:307-308)."""
    _need_cuda(x, w_gate_up, act)
    lib = load_module("gemm_tc")
    m = x.shape[0] if m is None else m
    two_i, k = w_gate_up.shape
    assert x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and act.dtype == torch.bfloat16
    assert x.shape[1] == k and act.shape[1] == two_i // 2 and x.stride(1) == 1 and w_gate_up.stride(1) == 1 and act.stride(1) == 1
    _check(lib, lib.abk_gemm_tc_swiglu(_p(x), _p(w_gate_up), _p(act), _i(m), _i(two_i // 2), _i(k), _ll(x.stride(0)),
                                       _ll(w_gate_up.stride(0)), _ll(act.stride(0)), _p(_Scratch.of(x.device).status),
                                       _stream()), "gemm_tc_swiglu")


def gemm_tc_qkv_takes(x, w_qkv, qkv, m, n_heads, n_kv_heads, head_dim, cache, q_norm, k_norm, cos, sin, rotary_dim, interleaved):
    """Whether the q/k/v product of a step takes the preparation of its heads (per-head norm, rotation, keys and values
    into the cache) into its epilogue: many rows, heads of 128, the rotation over the whole head in halves (or none),
    a cache that keeps every page."""
    tensors = [t for t in (q_norm, k_norm, cos, sin, cache.k, cache.v) if t is not None]
    return (m > 256 and head_dim == 128 and qkv.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
            and cache.ring_pages == 0 and w_qkv.shape[0] == (n_heads + 2 * n_kv_heads) * 128 == qkv.shape[1]
            and (cos is None or (rotary_dim == head_dim and not interleaved))
            and all(t.data_ptr() % 16 == 0 for t in tensors) and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0
            and all(t is None or t.dtype == torch.float32 for t in (q_norm, k_norm, cos, sin))
            and gemm_tc_takes(x, w_qkv, qkv))


def gemm_tc_qkv(x, w_qkv, qkv, n_heads, n_kv_heads, batch, q_norm, k_norm, eps, cos, sin, cache, m=None):
    """The q columns of qkv[:m] = the prepared q heads of x . w_qkv^T, and the prepared k and the v heads of every token
    that belongs to a sequence into the cache (cache.LayerKV): the q/k/v product of a prompt on the tcgen05 tensor
    cores with what stands between it and attention in its epilogue (src/model.c:299, 247-259). The k and v columns of
    qkv are not written."""
    _need_cuda(x, w_qkv, qkv)
    lib = load_module("gemm_tc")
    m = x.shape[0] if m is None else m
    assert x.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16 and qkv.dtype == torch.bfloat16
    assert x.shape[1] == w_qkv.shape[1] and x.stride(1) == 1 and w_qkv.stride(1) == 1 and qkv.stride(1) == 1
    assert cache.k.shape[1:] == (n_kv_heads, cache.tokens_per_page, 128) and cache.k.is_contiguous() and cache.v.is_contiguous()
    if cos is not None and batch.max_position >= cos.shape[0]:
        raise KernelError(f"position {batch.max_position} is beyond the rotary table of {cos.shape[0]} positions")
    _check(lib, lib.abk_gemm_tc_qkv(
        _p(x), _p(w_qkv), _p(qkv), _i(m), _i(n_heads), _i(n_kv_heads), _i(x.shape[1]), _ll(x.stride(0)), _ll(w_qkv.stride(0)),
        _ll(qkv.stride(0)), _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(q_norm), _p(k_norm), _f(eps or 0.0),
        _p(cos), _p(sin), _p(cache.k), _p(cache.v), _p(cache.page_table), _i(cache.table_width), _i(cache.tokens_per_page),
        _p(_Scratch.of(x.device).status), _stream()), "gemm_tc_qkv")


def argmax(logits, out, n_rows=None):
    """out[r] = index of the first maximum of logits[r] (src/main.c:31-36)."""
    _need_cuda(logits, out)
    lib = load_module("sampling")
    n = logits.shape[0] if n_rows is None else n_rows
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32 and out.numel() >= n
    sc = _Scratch.of(logits.device)
    if n > sc.argmax_rows:
        raise KernelRefused(f"argmax: {n} rows are more than the scratch of {sc.argmax_rows} rows")
    _check(lib, lib.abk_argmax(_p(logits), _ll(logits.stride(0)), _i(n), _i(logits.shape[1]), _p(out),
                               _p(sc.argmax_part), _p(sc.argmax_tickets), _stream()), "argmax")


def sample_topk(logits, temperature, top_k, rng_state, out, n_rows=None, rng_index=None):
    """Draw from the top_k logits at a temperature (src/main.c:39-56).

    rng_state int64 holds xorshift64 states; row r uses and advances rng_state[rng_index[r]]
    (rng_state[r] without rng_index).
    """
    _need_cuda(logits, rng_state, out, rng_index)
    lib = load_module("sampling")
    n = logits.shape[0] if n_rows is None else n_rows
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert rng_state.dtype == torch.int64 and out.numel() >= n
    assert rng_index is None or (rng_index.dtype == torch.int32 and rng_index.numel() >= n)
    assert rng_index is not None or rng_state.numel() >= n
    sc = _Scratch.of(logits.device)
    if n > sc.sample_rows:
        raise KernelRefused(f"sample_topk: {n} rows are more than the scratch of {sc.sample_rows} rows")
    _check(lib, lib.abk_sample_topk(_p(logits), _ll(logits.stride(0)), _i(n), _i(logits.shape[1]), _f(temperature),
                                    _i(top_k), _p(rng_state), _p(rng_index), _p(out), _p(sc.sample_part),
                                    _p(sc.sample_tickets), _stream()), "sample_topk")


def sample_all(logits, temperature, rng_state, out, n_rows=None, rng_index=None):
    """Draw from the whole vocabulary at a temperature (top_k = 0): p_j = exp((l_j - l_max) / temperature) over all j,
    walked in index order with abacus's generator (src/main.c:49-55 without the cut to 20 of src/main.c:41)."""
    _need_cuda(logits, rng_state, out, rng_index)
    lib = load_module("sampling")
    lib.abk_sample_all_scratch_bytes.restype = ctypes.c_longlong
    n = logits.shape[0] if n_rows is None else n_rows
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32 and out.numel() >= n
    assert rng_state.dtype == torch.int64
    assert rng_index is None or (rng_index.dtype == torch.int32 and rng_index.numel() >= n)
    assert rng_index is not None or rng_state.numel() >= n
    sc = _Scratch.of(logits.device)
    top = sc.grown("sample_all_top", n, torch.int32)
    sums = sc.grown("sample_all_sums", lib.abk_sample_all_scratch_bytes(_i(n), _i(logits.shape[1])), torch.uint8)
    argmax(logits, top, n)
    _check(lib, lib.abk_sample_all(_p(logits), _ll(logits.stride(0)), _i(n), _i(logits.shape[1]), _f(temperature), _p(top),
                                   _p(rng_state), _p(rng_index), _p(out), _p(sums), _stream()), "sample_all", kernels=2)


def attention(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, from_step=False, ws=None, lists=None,
              prepare=None, v_dim=None, keep_first=0, sink=None, exact_weights=False, row=None, chunk=None, softcap=None,
              gate=None):
    """Attention of a step: picks the kernel for the phase and sizes; every case the faster kernels
    do not take goes to the general one. lists: the step's tiles and work list for the prefill kernels
    (parts/attention_plan.py: AttentionLists); without them a step of several tokens runs on the general kernel.
    prepare: see attention_decode (only where attention_decode_prepares() said yes for this step).
    v_dim, keep_first, sink, exact_weights: see attention_generic and attention_window; the kernels for plain heads
    take none of them. gate: a gate per row and head (see attention_split) that the kernel may apply itself: returns True
    if it did (else the caller applies it)."""
    if chunk or softcap:  # the general kernel knows chunks and capped scores, and the prompt kernel with float32 weights
        assert prepare is None, "q, k and v must be prepared before this kernel"
        if (exact_weights and batch.is_decode and not from_step and ws is not None and qkv.dtype == torch.bfloat16
                and n_heads // n_kv_heads <= 16 and head_dim % 8 == 0):
            attention_split(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, ws, v_dim=v_dim,
                            keep_first=keep_first, sink=sink, row=row, chunk=chunk, softcap=softcap)
            return
        if (exact_weights and not batch.is_decode and not batch.any_continuation
                and attention_window_takes(qkv, head_dim, v_dim or head_dim, n_heads, n_kv_heads, row)):
            attention_window(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, v_dim=v_dim,
                             keep_first=keep_first, sink=sink, row=row, chunk=chunk, softcap=softcap)
            return
        attention_generic(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, from_step=from_step,
                          v_dim=v_dim, keep_first=keep_first, sink=sink, exact_weights=exact_weights, row=row, chunk=chunk,
                          softcap=softcap)
        return
    if (v_dim or head_dim) != head_dim or keep_first or sink is not None or exact_weights or row:
        assert prepare is None, "q, k and v must be prepared before these kernels"
        if (exact_weights and batch.is_decode and not from_step and ws is not None and qkv.dtype == torch.bfloat16
                and n_heads // n_kv_heads <= 16 and head_dim % 8 == 0):
            attention_split(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, ws, v_dim=v_dim,
                            keep_first=keep_first, sink=sink, row=row, gate=gate)  # one token a sequence: split along the keys
            return gate is not None
        if (exact_weights and not batch.is_decode and not batch.any_continuation
                and attention_window_takes(qkv, head_dim, v_dim or head_dim, n_heads, n_kv_heads, row)):
            attention_window(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, v_dim=v_dim,
                             keep_first=keep_first, sink=sink, row=row)  # whole prompts: keys from the step's rows
            return
        attention_generic(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, from_step=from_step,
                          v_dim=v_dim, keep_first=keep_first, sink=sink, exact_weights=exact_weights, row=row)
        return
    if (batch.is_decode and not from_step and ws is not None and qkv.dtype == torch.bfloat16
            and attention_decode_takes(n_heads, n_kv_heads, head_dim, cache)):
        attention_decode(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, ws, prepare=prepare)
        return
    assert prepare is None, "q, k and v must be prepared before any kernel but decode attention's"
    if (not batch.is_decode and not from_step and not window and qkv.dtype == torch.bfloat16 and lists is not None
          and attention_prefill_takes(head_dim, cache)):
        attention_prefill(qkv, out, n_heads, n_kv_heads, head_dim, scale, batch, cache, lists)
    else:
        attention_generic(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, from_step=from_step)


def attention_window_takes(qkv, head_dim, v_dim, n_heads, n_kv_heads, row=None):
    """Whether the tensor-core kernel for prompts with windows, sinks and values of their own size takes these sizes:
    bfloat16, heads and values multiples of 8 (values up to 128), every part of a row 16-byte aligned."""
    row = row or (n_heads + n_kv_heads) * head_dim + n_kv_heads * v_dim
    return (qkv.dtype == torch.bfloat16 and head_dim % 8 == 0 and 8 <= head_dim <= 256 and v_dim % 8 == 0
            and 8 <= v_dim <= 128 and row % 8 == 0 and qkv.data_ptr() % 16 == 0)


def attention_window(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, v_dim=None, keep_first=0, sink=None,
                     row=None, chunk=None, softcap=None):
    """Causal attention of whole prompts (every sequence of the step from its first token) on the warp-level tensor
    cores, keys and values from the step's own rows of qkv: an optional window that also keeps the first keep_first
    keys, an optional sink (float32 [n_heads]), values of v_dim, softmax weights in float32, keys seen only within the
    token's own chunk of `chunk` positions, scores capped at `softcap` (csrc/attention_window.cu)."""
    _need_cuda(qkv, out, sink)
    lib = load_module("attention_window")
    vd = v_dim or head_dim
    heads_size = (n_heads + n_kv_heads) * head_dim + n_kv_heads * vd
    row = row or heads_size
    n, n_seqs = batch.n_rows, batch.seq_slot.numel()
    assert qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and qkv.is_contiguous() and out.is_contiguous()
    assert qkv.shape[1] == row >= heads_size and out.shape[1] == n_heads * vd and qkv.shape[0] >= n and out.shape[0] >= n
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == n_heads)
    if batch.any_continuation:
        raise KernelRefused("attention_window reads keys from the step's rows: every sequence must start at position 0")
    max_tiles = (n + 63) // 64 + n_seqs
    _check(lib, lib.abk_attention_window(_p(qkv), _ll(row), _p(out), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(vd),
                                         _i(n_heads * head_dim), _i((n_heads + n_kv_heads) * head_dim), _f(scale),
                                         _i(window or 0), _i(keep_first or 0), _p(sink), _p(batch.seq_start), _i(n_seqs),
                                         _i(max_tiles), _i(chunk or 0), _f(softcap or 0.0), _stream()), "attention_window")


def attention_split(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, ws, v_dim=None, keep_first=0,
                    sink=None, row=None, max_keys=None, chunk=None, softcap=None, gate=None):
    """One new token per sequence against the paged cache with the general options (see attention_generic), split
    along the keys into parts of 128 that a second kernel folds (csrc/attention_split.cu); softmax weights float32.
    max_keys bounds the keys a row sees (by default the window and its kept keys, or the step's position bound).
    gate (of qkv's type, [rows, >= heads]): head h of row t is multiplied by sigmoid(gate[t, h]) where the parts are folded."""
    _need_cuda(qkv, out, sink, gate)
    assert gate is None or (gate.dtype == qkv.dtype and gate.stride(1) == 1 and gate.shape[1] >= n_heads)
    lib = load_module("attention_split")
    n, vd = batch.n_rows, v_dim or head_dim
    heads_size = (n_heads + n_kv_heads) * head_dim + n_kv_heads * vd
    row = row or heads_size
    assert qkv.is_contiguous() and qkv.shape[1] == row >= heads_size and out.is_contiguous() and out.dtype == qkv.dtype
    assert out.shape[1] == n_heads * vd and out.shape[0] >= n and cache.k.dtype == qkv.dtype and cache.v.shape[-1] == vd
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == n_heads)
    top = getattr(batch, "position_bound", None) or batch.max_len_after
    if batch.max_len_after > top:
        raise KernelError(f"a row at position {batch.max_len_after - 1} is beyond the bound {top}")
    if max_keys is None:
        max_keys = min(top, window + (keep_first or 0)) if window else top
        if chunk:
            max_keys = min(max_keys, chunk)
    n_parts = -(-max_keys // 128)
    parts = ws.get("attention_parts", (n * n_heads * n_parts * (vd + 2),), torch.float32)
    _check(lib, lib.abk_attention_split(
        _p(qkv), _ll(row), _p(out), _i(_dt(qkv)), _i(n), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(vd), _f(scale),
        _i(window or 0), _i(keep_first or 0), _p(sink), _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot),
        _p(cache.k), _p(cache.v), _p(cache.page_table), _i(cache.table_width), _i(cache.ring_pages),
        _i(cache.pinned_pages), _i(cache.tokens_per_page), _i(max_keys), _p(parts), _ll(parts.numel()), _i(chunk or 0),
        _f(softcap or 0.0), _p(gate), _ll(gate.stride(0) if gate is not None else 0), _stream()),
        "attention_split", kernels=2)


PREFILL_ON_MMA = False  # True: head size 128 too runs on the warp-level kernel (for comparison)


def attention_prefill_takes(head_dim, cache):
    return head_dim in (64, 128) and cache.tokens_per_page == 64 and cache.ring_pages == 0


def attention_prefill(qkv, out, n_heads, n_kv_heads, head_dim, scale, batch, cache, lists):
    """Causal attention of whole prompts (or any several tokens per sequence) against the paged bfloat16
    cache, on the tensor cores (src/model.c:197-211). No window. lists: the step's tiles of query rows and the
    work list of the kernel that halves long tiles (parts/attention_plan.py)."""
    _need_cuda(qkv, out)
    n = batch.n_rows
    row = (n_heads + 2 * n_kv_heads) * head_dim
    assert qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
    assert qkv.is_contiguous() and qkv.shape[1] == row and out.is_contiguous() and out.shape[1] == n_heads * head_dim
    assert cache.k.is_contiguous() and cache.v.is_contiguous()
    pool_rows = cache.k.shape[0] * cache.k.shape[1] * cache.k.shape[2]
    if head_dim == 128 and not PREFILL_ON_MMA:  # tcgen05: tiles of 128 query rows, scores and output in tensor memory
        lib = load_module("attention_tc")
        work = lists.work  # what each CTA does: whole tiles, long tiles twice
        sc = _Scratch.of(qkv.device)
        room = sc.attention_halves_pairs // n_heads
        if lists.n_halved > room:
            raise KernelRefused(f"attention_prefill_tc: the step halves {lists.n_halved} tiles, its scratch memory holds "
                                f"{room} for {n_heads} heads (the lists were made for another number of heads)")
        _check(lib, lib.abk_attention_prefill_tc(
            _p(qkv), _ll(row), _i(n), _p(out), _i(n_heads), _i(n_kv_heads), _i(head_dim), _f(scale), _p(work),
            _i(work.shape[0]), _i(room), _p(sc.attention_halves), _p(sc.attention_halves_tickets), _p(cache.k), _p(cache.v), _ll(pool_rows), _p(cache.page_table), _i(cache.table_width),
            _i(cache.tokens_per_page), _p(kernel_status(qkv.device)), _stream()), "attention_prefill_tc")
        return
    lib = load_module("attention_mma")
    tiles = lists.tiles(64)
    _check(lib, lib.abk_attention_prefill(
        _p(qkv), _ll(row), _i(n), _p(out), _i(n_heads), _i(n_kv_heads), _i(head_dim), _f(scale), _p(tiles),
        _i(tiles.shape[0]), _p(batch.seq_start), _p(batch.seq_pos0), _p(batch.seq_len_after), _p(batch.seq_slot),
        _p(cache.k), _p(cache.v), _ll(pool_rows), _p(cache.page_table), _i(cache.table_width),
        _i(cache.tokens_per_page), _p(kernel_status(qkv.device)), _stream()), "attention_prefill")


def attention_decode_prepares(qkv, n_heads, n_kv_heads, head_dim, cache, q_norm, k_norm, cos, sin, rotary_dim, interleaved):
    """Whether decode attention takes the q/k/v preparation (per-head norm, rotation, the new token's key and value
    into the cache) into its own kernel: on the tensor-core kernel, with the rotation over the whole head in halves
    (or none), and everything 16-byte aligned."""
    tensors = [t for t in (qkv, q_norm, k_norm, cos, sin, cache.k, cache.v) if t is not None]
    return (qkv.dtype == torch.bfloat16 and head_dim in (64, 128) and n_heads // n_kv_heads <= 16
            and attention_decode_takes(n_heads, n_kv_heads, head_dim, cache)
            and (cos is None or (rotary_dim == head_dim and not interleaved))
            and all(t.data_ptr() % 16 == 0 for t in tensors) and qkv.stride(0) % 8 == 0
            and all(t is None or t.dtype == torch.float32 for t in (q_norm, k_norm, cos, sin)))


def _attention_decode_mma(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, ws, max_positions,
                          prepare=None):
    lib = load_module("attention_decode_ring")
    n = batch.n_rows
    row = (n_heads + 2 * n_kv_heads) * head_dim
    assert qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
    assert qkv.is_contiguous() and qkv.shape[1] == row and out.is_contiguous() and out.shape[1] == n_heads * head_dim
    max_positions = max_positions or getattr(batch, "position_bound", None) or batch.max_len_after
    if batch.max_len_after > max_positions:
        raise KernelError(f"a row at position {batch.max_len_after - 1} is beyond the bound {max_positions}")
    pool_rows = cache.k.shape[0] * cache.k.shape[1] * cache.k.shape[2]
    if prepare is not None:
        cos = prepare["cos"]
        if cos is not None and batch.max_position >= cos.shape[0]:
            raise KernelError(f"position {batch.max_position} is beyond the rotary table of {cos.shape[0]} positions")
        _check(lib, lib.abk_attention_decode_ring_prepare(
            _p(qkv), _ll(row), _p(out), _i(n), _i(n_heads), _i(n_kv_heads), _i(head_dim), _f(scale), _i(window or 0),
            _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(cache.k), _p(cache.v), _ll(pool_rows),
            _p(cache.page_table), _i(cache.table_width), _i(cache.ring_pages), _i(cache.tokens_per_page),
            _i(max_positions), _p(prepare["q_norm"]), _p(prepare["k_norm"]), _f(prepare["eps"] or 0.0), _p(cos),
            _p(prepare["sin"]), _i(1 if prepare["keep"] else 0), _p(kernel_status(qkv.device)), _stream()),
            "attention_decode_mma")
        return
    _check(lib, lib.abk_attention_decode_ring(
        _p(qkv), _ll(row), _p(out), _i(n), _i(n_heads), _i(n_kv_heads), _i(head_dim), _f(scale), _i(window or 0),
        _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(cache.k), _p(cache.v), _ll(pool_rows),
        _p(cache.page_table), _i(cache.table_width), _i(cache.ring_pages), _i(cache.tokens_per_page),
        _i(max_positions), _p(kernel_status(qkv.device)), _stream()), "attention_decode_mma")


def attention_decode_takes(n_heads, n_kv_heads, head_dim, cache):
    group = n_heads // n_kv_heads
    smem = 4 * 64 * head_dim * 2 + 4 * group * (head_dim + 2) * 4 + 64
    return head_dim in (64, 128, 256) and cache.tokens_per_page == 64 and smem <= 200 * 1024


def attention_decode(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, ws, max_positions=None,
                     simt=False, prepare=None):
    """One new token per row against the paged bfloat16 cache, split along the keys (src/model.c:197-211).

    Head sizes 64 and 128 with groups of up to 16 query heads run on the tensor cores (mma.sync);
    head size 256, larger groups, or simt=True, on the CUDA cores.
    max_positions bounds every row's position + 1 (it sizes the grid and the scratch); by default
    the step's own maximum. A captured graph passes the bound it was captured for.
    prepare: dict(q_norm, k_norm, eps, cos, sin, keep) where attention_decode_prepares() says so: qkv is as the
    product left it, and the kernel norms and rotates q and k and (keep) writes the new key and value to the cache
    itself (src/model.c:247-259).
    """
    _need_cuda(qkv, out)
    if not simt and head_dim in (64, 128) and n_heads // n_kv_heads <= 16:
        return _attention_decode_mma(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, ws,
                                     max_positions, prepare)
    assert prepare is None, "only the tensor-core kernel prepares q, k and v itself"
    lib = load_module("attention_decode")
    lib.abk_attention_decode_scratch_floats.restype = ctypes.c_longlong
    n = batch.n_rows
    row = (n_heads + 2 * n_kv_heads) * head_dim
    assert qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
    assert qkv.is_contiguous() and qkv.shape[1] == row and out.is_contiguous() and out.shape[1] == n_heads * head_dim
    max_positions = max_positions or getattr(batch, "position_bound", None) or batch.max_len_after
    if batch.max_len_after > max_positions:
        raise KernelError(f"a row at position {batch.max_len_after - 1} is beyond the bound {max_positions}")
    chunks = -(-max_positions // 128)
    floats = lib.abk_attention_decode_scratch_floats(_i(n), _i(n_heads), _i(head_dim), _i(chunks))
    scratch = ws.get("attention_partials", (floats,), torch.float32)
    _check(lib, lib.abk_attention_decode(
        _p(qkv), _ll(row), _p(out), _i(n), _i(n_heads), _i(n_kv_heads), _i(head_dim), _f(scale), _i(window or 0),
        _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(cache.k), _p(cache.v), _p(cache.page_table),
        _i(cache.table_width), _i(cache.ring_pages), _i(cache.tokens_per_page), _i(max_positions), _p(scratch),
        _p(_attention_tickets(qkv.device, n * n_kv_heads)), _p(kernel_status(qkv.device)), _stream()),
        "attention_decode")


class _Scratch:
    """Per-device scratch of the kernels that need some: split-K partial tiles and their tickets,
    attention partials, and the status words a kernel sets when one of its bounded waits runs out."""
    _of_device = {}

    def __init__(self, device):
        self.device = device
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.argmax_rows = 4096
        self._made = {}

    def grown(self, name, count, dtype):
        """A buffer of at least `count` elements that is kept and only ever replaced by a larger one."""
        have = self._made.get(name)
        if have is None or have.numel() < count or have.dtype != dtype:
            have = self._made[name] = guards.empty(max(int(count), 1), dtype, self.device, what=f"scratch {name}")
        return have

    def _lazy(self, name, make):
        # each kernel's scratch is made at that kernel's first use, so that a model loads
        # (and compiles) only the kernel libraries it runs
        if name not in self._made:
            self._made[name] = make()
        return self._made[name]

    @property
    def gemm_floats(self):
        def make():
            lib = load_module("gemm_tc")
            lib.abk_gemm_tc_scratch_floats.restype = ctypes.c_longlong
            return guards.empty(lib.abk_gemm_tc_scratch_floats(), torch.float32, self.device, what="scratch of split K")
        return self._lazy("gemm_floats", make)

    @property
    def gemm_tickets(self):
        return self._lazy("gemm_tickets", lambda: guards.zeros(load_module("gemm_tc").abk_gemm_tc_scratch_tickets(),
                                                               torch.int32, self.device, what="tickets of split K"))

    @property
    def argmax_part(self):
        return self._lazy("argmax_part", lambda: guards.empty(
            self.argmax_rows * load_module("sampling").abk_argmax_slices() * 2, torch.float32, self.device, what="scratch of argmax"))

    sample_rows = 1024

    @property
    def sample_part(self):
        def make():
            lib = load_module("sampling")
            lib.abk_sample_topk_scratch_bytes.restype = ctypes.c_longlong
            return guards.empty(lib.abk_sample_topk_scratch_bytes(_i(self.sample_rows)), torch.uint8, self.device,
                                what="scratch of sampling")
        return self._lazy("sample_part", make)

    @property
    def sample_tickets(self):
        return self._lazy("sample_tickets", lambda: guards.zeros(self.sample_rows, torch.int32, self.device, what="tickets of sampling"))

    @property
    def argmax_tickets(self):
        return self._lazy("argmax_tickets", lambda: guards.zeros(self.argmax_rows, torch.int32, self.device, what="tickets of argmax"))

    attention_halves_pairs = 384  # (tile, head) pairs the prefill attention may halve in one launch (parts/attention_plan.py)

    @property
    def attention_halves(self):
        def make():
            lib = load_module("attention_tc")
            lib.abk_attention_prefill_tc_scratch_floats.restype = ctypes.c_longlong
            floats = lib.abk_attention_prefill_tc_scratch_floats(_i(self.attention_halves_pairs), _i(1))
            return guards.empty(floats, torch.float32, self.device, what="scratch of halved attention tiles")
        return self._lazy("attention_halves", make)

    @property
    def attention_halves_tickets(self):
        return self._lazy("attention_halves_tickets",
                          lambda: guards.zeros(2 * self.attention_halves_pairs, torch.int32, self.device,
                                               what="tickets of halved attention tiles"))

    @property
    def attention_tickets(self):
        return self._lazy("attention_tickets", lambda: guards.zeros(1 << 18, torch.int32, self.device, what="tickets of decode attention"))

    @classmethod
    def of(cls, device):
        key = (device.type, device.index)
        if key not in cls._of_device:
            cls._of_device[key] = cls(device)
        return cls._of_device[key]


def _attention_tickets(device, n):
    sc = _Scratch.of(device)
    if n > sc.attention_tickets.numel():
        raise KernelRefused(f"attention_decode: {n} (row, kv head) pairs are more than its {sc.attention_tickets.numel()} tickets")
    return sc.attention_tickets


def set_wait_limit_ns(ns, modules=("utility",)):
    """The limit of the bounded waits (on barriers, on another CTA's flag) of the named kernel libraries on the current
    device: a wait that has not been satisfied after `ns` nanoseconds gives up, the kernel sets its status word and
    returns. The libraries start at a quarter of a second."""
    for module in modules:
        lib = load_module(module)
        rc = lib.abk_set_wait_limit_ns(ctypes.c_ulonglong(int(ns)))
        if rc:
            raise KernelError(f"set_wait_limit_ns({module}): CUDA error {rc}")


def wait_that_runs_out(status, bit=4, word=1):
    """Launches the kernel whose one wait nothing can satisfy (csrc/utility.cu): after the utility library's limit it
    sets `bit` in status[word] and returns. For walking the way from a wait that ran out to the host's exception."""
    _need_cuda(status)
    lib = load_module("utility")
    assert status.dtype == torch.int32 and status.numel() > word
    _check(lib, lib.abk_wait_that_runs_out(ctypes.c_void_p(status.data_ptr() + 4 * word), _i(bit), _stream()),
           "wait_that_runs_out")


def kernel_status(device):
    """Status words of the device's kernels: all zero unless a kernel gave up on a wait."""
    return _Scratch.of(device).status


def gemm_tc_takes(x, w, out):
    """Whether the tensor-core kernel takes this product (else the CUDA-core kernel runs it):
    bfloat16 operands, K and both row pitches multiples of 8, 16-byte aligned."""
    k = w.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 8 == 0 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1)


def gemm_tc(x, w, out, m=None, tile_n=0, swap=-1, splits=0, persistent=-1):
    """out[:m] = x[:m] . w^T in bfloat16 on the tcgen05 tensor cores, float32 accumulation.

    tile_n, swap, splits and persistent pin the tile configuration (tests); 0 / -1 / 0 / -1 let the
    kernel choose.
    """
    _need_cuda(x, w, out)
    lib = load_module("gemm_tc")
    sc = _Scratch.of(x.device)
    m = x.shape[0] if m is None else m
    n, k = w.shape
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.shape[1] == k and out.shape[1] == n and x.shape[0] >= m and out.shape[0] >= m
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(lib, lib.abk_gemm_tc(_p(x), _p(w), _p(out), _i(_dt(out)), _i(m), _i(n), _i(k), _ll(x.stride(0)),
                                _ll(w.stride(0)), _ll(out.stride(0)), _p(sc.gemm_floats), _p(sc.gemm_tickets),
                                _p(sc.status), _i(tile_n), _i(swap), _i(splits), _i(persistent), _stream()), "gemm_tc")


# ------------------------------------------------------------------ streams (csrc/streams.cu)
def streams_step(x, y, connection, mult, enter, weight, eps, out, rows=None, n_rows=None):
    """What runs between two branches of a model whose residual stream is kept as several copies, x float32
    [tokens, s, d]: the write of the branch before, X'[t] = sum_s mix[s, t] X[s] + mult * leave[t] * y (y float32
    [tokens, d] or None: nothing pending; connection = (mix [s, s], leave [s])), stored in place; then the read for the
    branch after, u = sum_s enter[s] X'[s], and its norm, out = weight * u / sqrt(mean(u^2) + eps) (weight None:
    out = u). rows (int32): only those rows are made, into out[0:len(rows)], and x is left as it is."""
    _need_cuda(x, y, enter, weight, out, rows)
    lib = load_module("streams")
    n_tokens, s, d = x.shape
    n = n_rows if n_rows is not None else (rows.numel() if rows is not None else n_tokens)
    mix, leave = connection if y is not None else (None, None)
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape[-1] == d and out.shape[0] >= n
    assert y is None or (y.dtype == torch.float32 and y.is_contiguous() and y.shape[-1] == d and y.shape[0] >= (n if rows is None else 0))
    assert enter.dtype == torch.float32 and enter.numel() == s
    assert y is None or (mix.dtype == torch.float32 and mix.shape == (s, s) and mix.is_contiguous() and leave.numel() == s)
    assert weight is None or (weight.dtype == torch.float32 and weight.numel() == d)
    _check(lib, lib.abk_streams_step(_p(x), _p(y), _p(mix), _p(leave), _f(mult), _p(enter), _p(weight), _f(eps), _p(out),
                                     _i(_dt(out)), _p(rows), _i(n), _i(s), _i(d), _stream()), "streams_step")


def embed_pairs(batch, table, pairs, remembered, x, scale, buckets, mul_prev, mul_cur, status):
    """x[t, a] = table[token] * scale + pairs[(previous token * mul_prev + token * mul_cur) mod buckets] for every
    stream a (x float32 [tokens, s, d]); a sequence's first token takes row `buckets`; the token before a step's first
    row is the one its slot remembers (remembered int32 [slots]). pairs None: no second table."""
    _need_cuda(table, pairs, remembered, x, status)
    lib = load_module("streams")
    n, s, d = batch.n_rows, x.shape[1], x.shape[2]
    assert x.dtype == torch.float32 and x.is_contiguous() and x.shape[0] >= n and table.is_contiguous() and table.shape[1] == d
    assert pairs is None or (pairs.dtype == table.dtype and pairs.is_contiguous() and pairs.shape == (buckets + 1, d))
    assert pairs is None or remembered.dtype == torch.int32
    _check(lib, lib.abk_embed_pairs(_p(batch.tokens), _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot),
                                    _p(batch.seq_pos0), _p(table), _p(pairs), _i(_dt(table)), _p(remembered), _p(x),
                                    _f(scale), _i(n), _i(d), _i(table.shape[0]), _i(s), _ll(buckets), _ll(mul_prev),
                                    _ll(mul_cur), _p(status), _stream()), "embed_pairs")


def remember_tokens(batch, remembered):
    """remembered[slot] = the last token each sequence of the step brought."""
    _need_cuda(remembered)
    lib = load_module("streams")
    n_seqs = batch.seq_slot.numel()
    assert batch.seq_start.numel() >= n_seqs + 1 and remembered.dtype == torch.int32
    _check(lib, lib.abk_remember_tokens(_p(batch.tokens), _p(batch.seq_start), _p(batch.seq_slot), _i(n_seqs),
                                        _p(remembered), _stream()), "remember_tokens")


def embed_positions(batch, table, positions, x, keep, status):
    """x[t, a] = table[token] + positions[position] for every stream a (x float32 [tokens, s, d]): an embedding with a
    learned vector per position, not scaled. keep (float32 [tokens, d] or None) gets a copy of what the embedding leaves.
    A token or a position outside its table sets bit 0 of status and gives zeros."""
    _need_cuda(table, positions, x, keep, status)
    lib = load_module("streams")
    n, s, d = batch.n_rows, x.shape[1], x.shape[2]
    assert x.dtype == torch.float32 and x.is_contiguous() and x.shape[0] >= n and table.is_contiguous() and table.shape[1] == d
    assert positions.dtype == table.dtype and positions.is_contiguous() and positions.shape[1] == d
    assert keep is None or (keep.dtype == torch.float32 and keep.is_contiguous() and keep.shape[0] >= n and keep.shape[1] == d)
    _check(lib, lib.abk_embed_positions(_p(batch.tokens), _p(batch.token_seq), _p(batch.token_pos), _p(table), _p(positions),
                                        _i(_dt(table)), _p(x), _p(keep), _i(n), _i(d), _i(table.shape[0]),
                                        _i(positions.shape[0]), _i(s), _p(status), _stream()), "embed_positions")


def rejoin(x, kept, n):
    """x[t, a] += kept[t] for every stream a and t < n (x float32 [tokens, s, d], kept float32 [tokens, d])."""
    _need_cuda(x, kept)
    lib = load_module("streams")
    assert x.dtype == kept.dtype == torch.float32 and x.is_contiguous() and kept.is_contiguous()
    assert x.shape[0] >= n and kept.shape[0] >= n and x.shape[2] == kept.shape[1]
    _check(lib, lib.abk_rejoin(_p(x), _p(kept), _i(n), _i(x.shape[1]), _i(x.shape[2]), _stream()), "rejoin")


def normed_pair(a, b, weight_a, weight_b, out, n, eps, share):
    """out[t] = share * (weight_a * a[t] / rms(a[t]) + weight_b * b[t] / rms(b[t])), rms(v) = sqrt(mean(v^2) + eps): two
    branches that ran side by side, each normed over the width with a plain weight of its own. All float32 [tokens, d]."""
    _need_cuda(a, b, weight_a, weight_b, out)
    lib = load_module("streams")
    d = out.shape[1]
    for t in (a, b, out):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.shape[1] == d and t.shape[0] >= n
    assert weight_a.dtype == weight_b.dtype == torch.float32 and weight_a.numel() == weight_b.numel() == d
    _check(lib, lib.abk_normed_pair(_p(a), _p(b), _p(weight_a), _p(weight_b), _p(out), _i(n), _i(d), _f(eps), _f(share),
                                    _stream()), "normed_pair")


# ------------------------------------------------------------------ the delta-rule mixer (csrc/delta_rule.cu)
def short_conv(x, channels, weight, tail, out, batch, update_tail=False, plain=False):
    """out[t, c] = silu(sum_j weight[c, j] * x[position - (taps - 1 - j), c]) (plain: the sum without the SiLU) over the first `channels` columns of x
    (rows of any pitch), per sequence: zeros before its start, the slot's tail (float32 [slots, taps - 1, channels])
    before this step's rows. update_tail (only where every sequence of the step brings one token): the kernel leaves
    the slots' new tails itself, and short_conv_tail is not needed."""
    _need_cuda(x, weight, tail, out)
    assert not update_tail or batch.is_decode
    lib = load_module("delta_rule")
    n, taps = batch.n_rows, weight.shape[1]
    assert x.stride(1) == 1 and x.shape[1] >= channels and out.is_contiguous() and out.shape[1] == channels
    assert out.dtype == x.dtype and weight.dtype == torch.float32 and weight.shape == (channels, taps) and weight.is_contiguous()
    assert tail.dtype == torch.float32 and tail.shape[1:] == (max(taps - 1, 0), channels) and tail.is_contiguous()
    _check(lib, lib.abk_short_conv(_p(x), _ll(x.stride(0)), _p(out), _i(_dt(x)), _p(weight), _p(tail), _p(batch.token_seq),
                                   _p(batch.token_pos), _p(batch.seq_slot), _p(batch.seq_pos0), _i(n), _i(channels),
                                   _i(taps), _i(1 if update_tail else 0), _i(1 if plain else 0), _stream()), "short_conv")


def short_conv_tail(x, channels, taps, tail, batch):
    """The slots' tails after the step: each sequence's last taps - 1 inputs (from x's rows, and from the old tail
    where the step brought fewer)."""
    _need_cuda(x, tail)
    lib = load_module("delta_rule")
    n_seqs = batch.seq_slot.numel()
    assert x.stride(1) == 1 and tail.dtype == torch.float32 and tail.is_contiguous()
    _check(lib, lib.abk_short_conv_tail(_p(x), _ll(x.stride(0)), _i(_dt(x)), _p(tail), _p(batch.seq_start),
                                        _p(batch.seq_slot), _p(batch.seq_pos0), _i(n_seqs), _i(channels), _i(taps),
                                        _stream()), "short_conv_tail")


DELTA_CHUNK = 64  # tokens of a chunk of the chunked form (one decay a head)


def delta_scan(qkv, decay_in, beta_in, a_log, dt_bias, state, out, batch, n_heads, n_kv_heads, key_dim, value_dim, ws,
               per_head=False, chunks=False):
    """The gated delta rule over every sequence of the step, token by token, from and into the slots' states (float32
    [slots, heads, value, key]). qkv [tokens, 2 * kv_heads * key + heads * value]: q, k and v after their convolution;
    decay_in float32 [tokens, heads * key] (rows of any pitch) before bias and softplus; beta_in [tokens, >= heads] (rows of any pitch)
    before the sigmoid; out float32 [tokens, heads * value], not yet normed. per_head: one decay for all key channels of a
    head; decay_in is then [tokens, >= heads] of qkv's type and dt_bias [heads]. Two kernels: every (token, head) is
    prepared in parallel into scratch memory from ws (a parts.Workspace), then the sequences are walked. chunks (with
    per_head, for steps that bring prompts): the walk goes in chunks of 64 tokens, a triangular system a chunk solved
    beside the others and four products a chunk along the sequence (three kernels)."""
    _need_cuda(qkv, decay_in, beta_in, a_log, dt_bias, state, out)
    lib = load_module("delta_rule")
    lib.abk_delta_scan_scratch.restype = ctypes.c_longlong
    n, n_seqs = batch.n_rows, batch.seq_slot.numel()
    assert qkv.is_contiguous() and qkv.shape[1] == 2 * n_kv_heads * key_dim + n_heads * value_dim and qkv.shape[0] >= n
    if per_head:
        assert decay_in.dtype == qkv.dtype and decay_in.stride(1) == 1 and decay_in.shape[1] >= n_heads and dt_bias.numel() == n_heads
    else:
        assert decay_in.dtype == torch.float32 and decay_in.stride(1) == 1 and decay_in.shape[1] == n_heads * key_dim
        assert dt_bias.numel() == n_heads * key_dim
    assert beta_in.dtype == qkv.dtype and beta_in.stride(1) == 1 and beta_in.shape[1] >= n_heads
    assert a_log.dtype == torch.float32 and dt_bias.dtype == torch.float32 and a_log.numel() == n_heads
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (n_heads, value_dim, key_dim)
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape[1] == n_heads * value_dim
    records = ws.get("delta_records", (int(lib.abk_delta_scan_scratch(_i(n), _i(n_heads), _i(key_dim), _i(value_dim))),),
                     torch.float32)
    if chunks:
        assert per_head, "the chunked form takes one decay a head"
        max_chunks = -(-n // DELTA_CHUNK) + n_seqs
        work = ws.get("delta_chunks", (max_chunks * n_heads * (DELTA_CHUNK * DELTA_CHUNK + 2 * DELTA_CHUNK),), torch.float32)
        _check(lib, lib.abk_delta_chunks(
            _p(qkv), _ll(qkv.stride(0)), _i(_dt(qkv)), _p(decay_in), _ll(decay_in.stride(0)), _p(beta_in),
            _ll(beta_in.stride(0)), _p(a_log), _p(dt_bias), _p(state), _p(out), _p(batch.token_seq), _p(batch.seq_start),
            _p(batch.seq_slot), _i(n), _i(n_seqs), _i(n_heads), _i(n_kv_heads), _i(key_dim), _i(value_dim), _p(records),
            _ll(records.numel()), _i(max_chunks), _p(work), _ll(work.numel()), _stream()), "delta_chunks", kernels=3)
        return
    _check(lib, lib.abk_delta_scan(_p(qkv), _ll(qkv.stride(0)), _i(_dt(qkv)), _p(decay_in), _ll(decay_in.stride(0)),
                                   _i(1 if per_head else 0), _p(beta_in), _ll(beta_in.stride(0)), _p(a_log), _p(dt_bias), _p(state), _p(out), _p(batch.token_seq),
                                   _p(batch.seq_start), _p(batch.seq_slot), _i(n), _i(n_seqs), _i(n_heads), _i(n_kv_heads),
                                   _i(key_dim), _i(value_dim), _p(records), _ll(records.numel()), _stream()),
           "delta_scan", kernels=2)


def gated_head_norm(o, gate, weight, out, n_tokens, n_heads, value_dim, eps, silu=False):
    """out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * weight * sigmoid(gate[t, h]) (silu: times gate * sigmoid(gate));
    o float32 [tokens, heads * value]; gate float32 or of out's type, [tokens, heads * value] (rows of any pitch); weight
    float32 [value], shared by the heads, or [heads * value]."""
    _need_cuda(o, gate, weight, out)
    lib = load_module("delta_rule")
    assert o.dtype == torch.float32 and gate.dtype in (torch.float32, out.dtype) and weight.dtype == torch.float32
    assert o.is_contiguous() and gate.stride(1) == 1 and out.is_contiguous() and weight.numel() in (value_dim, n_heads * value_dim)
    assert o.shape[1] == gate.shape[1] == out.shape[1] == n_heads * value_dim
    _check(lib, lib.abk_gated_head_norm(_p(o), _p(gate), _ll(gate.stride(0)), _i(0 if gate.dtype == torch.float32 else 1), _p(weight),
                                        _p(out), _i(_dt(out)), _i(n_tokens), _i(n_heads), _i(value_dim), _f(eps),
                                        _i(1 if silu else 0), _i(1 if weight.numel() != value_dim else 0), _stream()),
           "gated_head_norm")


# ------------------------------------------------------------------ latent attention (csrc/latent.cu)
def latent_prep(proj, down_at, n_heads, dim, rot, rank, rot_dims, norm_w, eps, cos, sin, q_dst, q_head, q_rot_at, copy_plain,
                cache, batch, interleaved=True):
    """What stands between the projections of a latent-attention layer and its attention kernel, per token: the
    latent c = norm_w * z / sqrt(mean(z^2) + eps) over the first `rank` columns of the down-projection (proj[:,
    down_at:]), the rotation (pairs (2i, 2i+1), or with interleaved False (i, i + rot_dims / 2), of the first rot_dims
    elements) of the shared key part behind it and of
    every query head's rotated part (proj[:, h * (dim + rot) + dim:]), the row [c | r | zeros] written to the cache
    (cache: a cache.LayerKV whose rows hold at least rank + rot elements; None: the entry reads another's cache), and
    the query parts put into q_dst: head h of a row at h * q_head, its rotated part at + q_rot_at (zeros behind it up
    to the head's end), its plain part (copy_plain) at + 0."""
    _need_cuda(proj, norm_w, cos, sin, q_dst)
    lib = load_module("latent")
    n = batch.n_rows
    assert proj.stride(1) == 1 and q_dst.stride(1) == 1 and q_dst.dtype == proj.dtype and proj.shape[0] >= n
    assert cos is None or (cos.dtype == torch.float32 and cos.shape == sin.shape and cos.shape[1] == rot_dims // 2)
    if cos is not None and batch.max_position >= cos.shape[0]:
        raise KernelError(f"position {batch.max_position} is beyond the rotary table of {cos.shape[0]} positions")
    if cos is None:
        rot_dims = 0
    if cache is not None:
        assert cache.k.dtype == proj.dtype and cache.k.shape[1] == 1 and cache.ring_pages == 0 and cache.k.is_contiguous()
        assert norm_w.dtype == torch.float32 and norm_w.numel() == rank
    _check(lib, lib.abk_latent_prep(
        _p(proj), _ll(proj.stride(0)), _i(_dt(proj)), _i(n), _i(down_at), _i(n_heads), _i(dim), _i(rot), _i(rank),
        _i(rot_dims), _i(1 if interleaved else 0), _p(norm_w), _f(eps), _p(cos), _p(sin), _p(q_dst), _ll(q_dst.stride(0)),
        _i(q_head), _i(q_rot_at),
        _i(1 if copy_plain else 0), _p(cache.k if cache is not None else None),
        _i(cache.k.shape[-1] if cache is not None else 0), _p(cache.page_table if cache is not None else None),
        _i(cache.table_width if cache is not None else 0), _i(cache.tokens_per_page if cache is not None else 1),
        _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _stream()), "latent_prep")


def head_product(x, x_head, w, out, o_head, n, gate=None):
    """out[t, h * o_head + o] = sum_i w[h, o, i] * x[t, h * x_head + i] for t < n: a product per head with a matrix of
    its own, w [heads, outs, in]; x, w and out of one type, rows of any pitch. gate (of their type, [rows, >= heads]):
    head h of row t is multiplied by sigmoid(gate[t, h])."""
    _need_cuda(x, w, out)
    lib = load_module("latent")
    heads, outs, inner = w.shape
    assert x.dtype == w.dtype == out.dtype and w.is_contiguous() and x.stride(1) == 1 and out.stride(1) == 1
    assert x.shape[0] >= n and out.shape[0] >= n and x_head >= inner and o_head >= outs
    assert x.shape[1] >= (heads - 1) * x_head + inner and out.shape[1] >= (heads - 1) * o_head + outs
    assert gate is None or (gate.dtype == x.dtype and gate.stride(1) == 1 and gate.shape[1] >= heads and gate.shape[0] >= n)
    _check(lib, lib.abk_head_product(_p(x), _ll(x.stride(0)), _i(x_head), _p(w), _p(out), _ll(out.stride(0)), _i(o_head),
                                     _i(_dt(x)), _i(n), _i(heads), _i(inner), _i(outs), _p(gate),
                                     _ll(gate.stride(0) if gate is not None else 0), _stream()), "head_product")


def latent_rows(cache, rows, count, batch):
    """rows[t, :count] = the first `count` elements of the cache row of the step's token t (cache: a cache.LayerKV
    with one kv head)."""
    _need_cuda(rows)
    lib = load_module("latent")
    assert rows.dtype == cache.k.dtype and rows.stride(1) == 1 and rows.shape[0] >= batch.n_rows and cache.ring_pages == 0
    _check(lib, lib.abk_latent_rows(_p(cache.k), _i(cache.k.shape[-1]), _p(cache.page_table), _i(cache.table_width),
                                    _i(cache.tokens_per_page), _p(rows), _ll(rows.stride(0)), _i(count), _i(_dt(rows)),
                                    _i(batch.n_rows), _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot),
                                    _stream()), "latent_rows")


def spread_shared(shared, keys, k_head, at, count, heads, n):
    """keys[t, h * k_head + at + i] = shared[t, i] for every head h and i < count: a key part that the heads share,
    copied behind each head's own part."""
    _need_cuda(shared, keys)
    lib = load_module("latent")
    assert shared.dtype == keys.dtype and shared.stride(1) == 1 and keys.stride(1) == 1
    assert shared.shape[1] >= count and keys.shape[1] >= (heads - 1) * k_head + at + count
    _check(lib, lib.abk_spread_shared(_p(shared), _ll(shared.stride(0)), _p(keys), _ll(keys.stride(0)), _i(k_head), _i(at),
                                      _i(count), _i(heads), _i(_dt(keys)), _i(n), _stream()), "spread_shared")


def attention_values_in_keys(q, out, n_heads, head_dim, v_dim, scale, batch, cache, sink=None, ws=None):
    """Causal attention of every token of the step over a cache with one kv head whose values are the first v_dim
    elements of its keys (latent rows), float32 softmax weights, an optional sink. q [tokens, n_heads * head_dim], out
    [tokens, n_heads * v_dim]. A step of one token a sequence in bfloat16 with rows of up to 256
    runs split along the keys (csrc/attention_split.cu), everything else on the general kernel."""
    _need_cuda(q, out, sink)
    n = batch.n_rows
    assert q.is_contiguous() and q.shape[1] == n_heads * head_dim and out.is_contiguous() and out.dtype == q.dtype
    assert out.shape[1] == n_heads * v_dim and cache.k.dtype == q.dtype and cache.k.shape[1:] == (1, cache.tokens_per_page, head_dim)
    assert cache.values_in_keys and cache.ring_pages == 0 and v_dim <= head_dim
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == n_heads)
    if batch.is_decode and ws is not None and q.dtype == torch.bfloat16 and head_dim % 8 == 0 and head_dim <= 256:
        lib = load_module("attention_split")
        top = getattr(batch, "position_bound", None) or batch.max_len_after
        if batch.max_len_after > top:
            raise KernelError(f"a row at position {batch.max_len_after - 1} is beyond the bound {top}")
        n_parts = -(-top // 128)
        parts = ws.get("attention_parts", (n * n_heads * n_parts * (v_dim + 2),), torch.float32)
        _check(lib, lib.abk_attention_split_values_in_keys(
            _p(q), _ll(q.shape[1]), _p(out), _i(_dt(q)), _i(n), _i(n_heads), _i(1), _i(head_dim), _i(v_dim), _f(scale),
            _p(sink), _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(cache.k), _p(cache.page_table),
            _i(cache.table_width), _i(cache.tokens_per_page), _i(top), _p(parts), _ll(parts.numel()), _stream()),
            "attention_split", kernels=2)
        return
    lib = load_module("attention_generic")
    _check(lib, lib.abk_attention_values_in_keys(
        _p(q), _ll(q.shape[1]), _p(out), _i(_dt(q)), _i(n), _i(n_heads), _i(1), _i(head_dim), _f(scale),
        _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(batch.seq_start), _p(batch.seq_pos0), _p(cache.k),
        _p(cache.page_table), _i(cache.table_width), _i(cache.tokens_per_page), _i(v_dim), _p(sink), _i(1), _stream()),
        "attention")


# ------------------------------------------------------------------ linear attention with a decay (csrc/lightning.cu)
def lightning_scan(proj, q_at, k_at, v_at, n_heads, dim, vdim, decay, state, out, batch):
    """Per head S <- decay_h S + k v^T, o = S^T q over every sequence of the step, token by token, from and into the
    slots' states (float32 [slots, heads, dim, vdim]). q, k (heads x dim) and v (heads x vdim) are the SiLU of the
    columns of proj from q_at, k_at and v_at on; out float32 [tokens, heads * vdim]."""
    _need_cuda(proj, decay, state, out)
    lib = load_module("lightning")
    n_seqs = batch.seq_slot.numel()
    assert proj.stride(1) == 1 and proj.shape[0] >= batch.n_rows and out.dtype == torch.float32 and out.is_contiguous()
    assert out.shape[1] == n_heads * vdim and decay.dtype == torch.float32 and decay.numel() == n_heads
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (n_heads, dim, vdim)
    assert batch.seq_start.numel() >= n_seqs + 1
    _check(lib, lib.abk_lightning_scan(_p(proj), _ll(proj.stride(0)), _i(_dt(proj)), _i(q_at), _i(k_at), _i(v_at),
                                       _i(n_heads), _i(dim), _i(vdim), _p(decay), _p(state), _p(out), _p(batch.seq_start),
                                       _p(batch.seq_slot), _i(n_seqs), _stream()), "lightning_scan")


LIGHTNING_CHUNK = 64  # tokens of a chunk of the chunked form


def lightning_chunks(proj, q_at, k_at, v_at, n_heads, dim, vdim, decay, state, out, batch, ws):
    """lightning_scan for steps that bring prompts: the same recurrence in chunks of 64 tokens, the chunks' sums and
    outputs side by side and only the states between chunks along the sequence (csrc/lightning.cu). ws: a
    parts.Workspace for the chunks' sums."""
    _need_cuda(proj, decay, state, out)
    lib = load_module("lightning")
    n_seqs = batch.seq_slot.numel()
    assert proj.stride(1) == 1 and proj.shape[0] >= batch.n_rows and out.dtype == torch.float32 and out.is_contiguous()
    assert out.shape[1] == n_heads * vdim and decay.dtype == torch.float32 and decay.numel() == n_heads
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (n_heads, dim, vdim)
    assert batch.seq_start.numel() >= n_seqs + 1
    max_chunks = -(-batch.n_rows // LIGHTNING_CHUNK) + n_seqs
    sums = ws.get("lightning_sums", (max_chunks * n_heads * dim * vdim,), torch.float32)
    _check(lib, lib.abk_lightning_chunks(_p(proj), _ll(proj.stride(0)), _i(_dt(proj)), _i(q_at), _i(k_at), _i(v_at),
                                         _i(n_heads), _i(dim), _i(vdim), _p(decay), _p(state), _p(out), _p(batch.seq_start),
                                         _p(batch.seq_slot), _i(n_seqs), _i(max_chunks), _p(sums), _ll(sums.numel()),
                                         _stream()), "lightning_chunks", kernels=3)


def gated_row_norm(o, gate, weight, out, eps, batch):
    """out[t] = weight * o[t] / sqrt(mean(o[t]^2) + eps) * sigmoid(gate[t]) over a token's whole row; o float32
    [tokens, width], gate of out's type (rows of any pitch), weight float32 [width]; rows of padding become zeros."""
    _need_cuda(o, gate, weight, out)
    lib = load_module("lightning")
    n, width = batch.n_rows, o.shape[1]
    assert o.dtype == torch.float32 and o.is_contiguous() and out.is_contiguous() and out.shape[1] == width
    assert gate.dtype == out.dtype and gate.stride(1) == 1 and gate.shape[1] >= width and weight.dtype == torch.float32
    assert weight.numel() == width and o.shape[0] >= n and out.shape[0] >= n
    _check(lib, lib.abk_gated_row_norm(_p(o), _p(gate), _ll(gate.stride(0)), _p(weight), _p(out), _i(_dt(out)), _i(n),
                                       _i(width), _f(eps), _p(batch.token_seq), _stream()), "gated_row_norm")


# ------------------------------------------------------------------ a matrix memory with exponential gates (csrc/matrix_memory.cu)
def matrix_memory_blocks(value_dim):
    """How many copies of n and m a head's state holds (one per CTA that walks the head)."""
    return int(load_module("matrix_memory").abk_matrix_memory_blocks(_i(value_dim)))


MATRIX_MEMORY_CHUNK = 64  # tokens of a chunk of the chunked form


def matrix_memory(proj, q_at, k_at, v_at, gates, bias_i, bias_f, cap, denom_eps, n_heads, key_dim, value_dim, state_c,
                  state_n, state_m, out, batch, ws=None):
    """Per head, token by token over every sequence of the step, from and into the slots' states:
        i = cap tanh((zi + bi) / cap);  f = logsigmoid(cap tanh((zf + bf) / cap));  m' = max(f + m, i)
        C' = e^(f + m - m') C + e^(i - m') k v^T;  n' likewise with k alone;  o = C'^T q / (max(|n' . q|, e^-m') + denom_eps)
    q (times key_dim^-1/2 here), k (heads x key) and v (heads x value) are the columns of proj from q_at, k_at and v_at on;
    gates float32 [tokens, 2 * heads] (rows of any pitch): zi, then zf. States float32: state_c [slots, heads, value, key],
    state_n [slots, heads, blocks, key], state_m [slots, heads, blocks] with blocks = matrix_memory_blocks(value_dim).
    out float32 [tokens, heads * value], not yet normed. ws (a parts.Workspace): the same recurrence in chunks of 64
    tokens, for steps that bring prompts: the chunks' sums and outputs side by side and only the states between chunks
    along the sequence (three launches)."""
    _need_cuda(proj, gates, bias_i, bias_f, state_c, state_n, state_m, out)
    lib = load_module("matrix_memory")
    n_seqs = batch.seq_slot.numel()
    blocks = matrix_memory_blocks(value_dim)
    assert proj.stride(1) == 1 and proj.shape[0] >= batch.n_rows and out.dtype == torch.float32 and out.is_contiguous()
    assert out.shape[1] == n_heads * value_dim and gates.dtype == torch.float32 and gates.stride(1) == 1
    assert gates.shape[1] >= 2 * n_heads and bias_i.dtype == bias_f.dtype == torch.float32
    assert bias_i.numel() == bias_f.numel() == n_heads
    for st, shape in ((state_c, (n_heads, value_dim, key_dim)), (state_n, (n_heads, blocks, key_dim)), (state_m, (n_heads, blocks))):
        assert st.dtype == torch.float32 and st.is_contiguous() and tuple(st.shape[1:]) == shape
    assert batch.seq_start.numel() >= n_seqs + 1
    if ws is not None:
        max_chunks = -(-batch.n_rows // MATRIX_MEMORY_CHUNK) + n_seqs
        work = ws.get("memory_chunks", (max_chunks * n_heads * (value_dim * key_dim + key_dim + 4),), torch.float32)
        _check(lib, lib.abk_matrix_memory_chunks(
            _p(proj), _ll(proj.stride(0)), _i(_dt(proj)), _i(q_at), _i(k_at), _i(v_at), _p(gates), _ll(gates.stride(0)),
            _p(bias_i), _p(bias_f), _f(cap), _f(denom_eps), _f(float(key_dim) ** -0.5), _i(n_heads), _i(key_dim),
            _i(value_dim), _p(state_c), _p(state_n), _p(state_m), _p(out), _p(batch.seq_start), _p(batch.seq_slot),
            _i(n_seqs), _i(max_chunks), _p(work), _ll(work.numel()), _stream()), "matrix_memory_chunks", kernels=3)
        return
    _check(lib, lib.abk_matrix_memory(_p(proj), _ll(proj.stride(0)), _i(_dt(proj)), _i(q_at), _i(k_at), _i(v_at), _p(gates),
                                      _ll(gates.stride(0)), _p(bias_i), _p(bias_f), _f(cap), _f(denom_eps),
                                      _f(float(key_dim) ** -0.5), _i(n_heads), _i(key_dim), _i(value_dim), _p(state_c),
                                      _p(state_n), _p(state_m), _p(out), _p(batch.seq_start), _p(batch.seq_slot), _i(n_seqs),
                                      _stream()), "matrix_memory")


# ------------------------------------------------------------------ routed experts (csrc/moe.cu)
RELU_SQUARED = 1
SILU_GATED = 2  # the matrix holds gate rows, then up rows: silu(gate . x) * (up . x)


def moe_route(x, router, top, batch, pair_expert, pair_weight, softmax_chosen=False, always=None, softmax_all=False,
              correction=None, weight_scale=1.0, n_real=None):
    """Per token the `top` experts with the largest router logits (router float32 [experts, d], x as stored) and their
    weights, sigmoid(logit) or the softmax over the chosen; pair token * top + k is the token's k-th choice
    (pair_expert int32, -1 for padding rows; pair_weight float32). always (an expert's index): every token has top + 1
    pairs, the last that expert with weight 1. softmax_all: s = softmax over all router outputs, the choice goes by
    s + correction (float32 [outputs] or None), the weight is s * weight_scale. n_real: router outputs from there on stand
    for experts that return their input; such a pair carries -2 - (output - n_real)."""
    _need_cuda(x, router, pair_expert, pair_weight, correction)
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == router.shape[0])
    lib = load_module("moe")
    n, (experts, d) = batch.n_rows, router.shape
    assert router.dtype == torch.float32 and router.is_contiguous() and x.stride(1) == 1 and x.shape[1] == d
    assert pair_expert.dtype == torch.int32 and pair_weight.dtype == torch.float32
    per = top + (0 if always is None else 1)
    assert pair_expert.numel() >= n * per and pair_weight.numel() >= n * per
    _check(lib, lib.abk_moe_route(_p(x), _ll(x.stride(0)), _i(_dt(x)), _p(router), _i(n), _i(d), _i(experts), _i(top),
                                  _i(2 if softmax_all else 1 if softmax_chosen else 0), _i(-1 if always is None else always),
                                  _p(batch.token_seq), _p(pair_expert), _p(pair_weight), _p(correction), _f(weight_scale),
                                  _i(experts if n_real is None else n_real), _stream()), "moe_route")


def routed_product(x, pairs_per_row, w, pair_expert, pair_scale, out, n_pairs, activation=0):
    """out[p] = act(w[pair_expert[p]] (pair_scale[p] * x[p // pairs_per_row])) for p < n_pairs: a product whose matrix,
    w [experts, outs, in], is chosen per row. pair_scale None: no scale; with one the scaled input is rounded to x's
    type first. out of x's type or float32. activation: 0 none, RELU_SQUARED, or SILU_GATED (w [experts, 2 * outs, in]: gate
    rows, then up rows). Pairs whose expert is negative give zeros."""
    _need_cuda(x, w, pair_expert, pair_scale, out)
    lib = load_module("moe")
    experts, outs, inner = w.shape
    if activation == SILU_GATED:
        assert outs % 2 == 0
        outs //= 2
    assert x.dtype == w.dtype and w.is_contiguous() and x.stride(1) == 1 and x.shape[1] == inner
    assert out.stride(1) == 1 and out.shape[1] == outs and out.shape[0] >= n_pairs and out.dtype in (x.dtype, torch.float32)
    _check(lib, lib.abk_routed_product(_p(x), _ll(x.stride(0)), _i(pairs_per_row), _i(_dt(x)), _p(w), _p(pair_expert),
                                       _p(pair_scale), _p(out), _ll(out.stride(0)),
                                       _i(1 if out.dtype == torch.float32 and x.dtype != torch.float32 else 0),
                                       _i(activation), _i(n_pairs), _i(inner), _i(outs), _stream()), "routed_product")


def moe_combine(pairs, out, n, top, add):
    """out[t] = (out[t] if add else 0) + sum over k of pairs[t * top + k], in the order of k; all float32."""
    _need_cuda(pairs, out)
    lib = load_module("moe")
    d = out.shape[1]
    assert pairs.dtype == out.dtype == torch.float32 and pairs.is_contiguous() and out.is_contiguous()
    assert pairs.shape[1] == d and pairs.shape[0] >= n * top and out.shape[0] >= n
    _check(lib, lib.abk_moe_combine(_p(pairs), _p(out), _i(n), _i(d), _i(top), _i(1 if add else 0), _stream()), "moe_combine")


def moe_combine_weighted(pairs, weight, expert, x, out, n, top, place=None):
    """out[t] = sum over k of weight[t * top + k] * (pairs[t * top + k], or x[t] where expert[t * top + k] <= -2: an expert
    that returns its input), in the order of k; pairs, weight and out float32, x as stored. place int32: the rows of
    `pairs` lie sorted by expert, pair p's at place[p]."""
    _need_cuda(pairs, weight, expert, x, out)
    lib = load_module("moe")
    d = out.shape[1]
    assert pairs.dtype == out.dtype == weight.dtype == torch.float32 and pairs.is_contiguous() and out.is_contiguous()
    assert pairs.shape[1] == d and out.shape[0] >= n and x.stride(1) == 1 and x.shape[1] == d
    assert expert.dtype == torch.int32
    if place is None:
        assert pairs.shape[0] >= n * top
    else:
        _need_cuda(place)
        assert place.dtype == torch.int32 and place.numel() >= n * top
    _check(lib, lib.abk_moe_combine_weighted(_p(pairs), _p(weight), _p(expert), _p(x), _ll(x.stride(0)), _i(_dt(x)), _p(out),
                                             _i(n), _i(d), _i(top), _p(place) if place is not None else ctypes.c_void_p(0),
                                             _stream()), "moe_combine_weighted")


def relu_squared(x, n):
    """x[:n] = max(x, 0)^2 in place (x contiguous)."""
    _need_cuda(x)
    lib = load_module("moe")
    assert x.is_contiguous()
    _check(lib, lib.abk_relu_squared(_p(x), _i(_dt(x)), _ll(n * x.shape[1]), _stream()), "relu_squared")


# ------------------------------------------------------------------ routed experts over many rows (csrc/gemm_grouped.cu)
GROUPED_ROWS = 128  # rows of a tile of the grouped product: an expert's run of sorted rows is padded to whole tiles


def grouped_tiles(n_pairs, experts):
    """Row tiles that hold n_pairs pairs sorted by expert, whatever the routing."""
    return -(-n_pairs // GROUPED_ROWS) + experts


def grouped_takes(x, up, down):
    """Whether the tensor-core products by expert take these: bfloat16, inner sizes multiples of 8, 16-byte aligned."""
    return (x.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 and up.shape[2] % 8 == 0 and down.shape[2] % 8 == 0
            and up.data_ptr() % 16 == 0 and down.data_ptr() % 16 == 0)


def moe_sort(x, pairs_per_row, pair_expert, pair_scale, n_pairs, experts, scratch, place, tile_expert, sorted_rows):
    """Pairs sorted by expert, each expert's run padded to whole tiles of 128 rows: place[p] int32 is pair p's row in
    the sorted order (-1 for pairs of padding rows), tile_expert[t] int32 the expert of row tile t (-1 beyond the used
    ones), sorted_rows bfloat16 [tiles * 128, d] the pairs' input rows x[p // pairs_per_row], times pair_scale[p]
    where given. scratch int32 [2 * experts + n_pairs]."""
    _need_cuda(x, pair_expert, pair_scale, scratch, place, tile_expert, sorted_rows)
    lib = load_module("gemm_grouped")
    d, max_tiles = x.shape[1], tile_expert.numel()
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and sorted_rows.dtype == torch.bfloat16 and sorted_rows.is_contiguous()
    assert sorted_rows.shape == (max_tiles * GROUPED_ROWS, d) and scratch.dtype == torch.int32 and scratch.numel() >= 2 * experts + n_pairs
    assert place.dtype == torch.int32 and place.numel() >= n_pairs and tile_expert.dtype == torch.int32
    counts, first, rank = scratch[:experts], scratch[experts:2 * experts], scratch[2 * experts:]
    _check(lib, lib.abk_moe_sort(_p(x), _ll(x.stride(0)), _i(pairs_per_row), _p(pair_expert), _p(pair_scale), _i(n_pairs),
                                 _i(experts), _i(d), _p(counts), _p(rank), _p(first), _p(place), _p(tile_expert),
                                 _i(max_tiles), _p(sorted_rows), _stream()), "moe_sort", kernels=3)


def gemm_grouped(x, w, out, tile_expert, activation=0):
    """out[p] = act(w[tile_expert[p // 128]] x[p]) for the sorted rows x bfloat16 [tiles * 128, K] on the tcgen05 tensor
    cores; w bfloat16 [experts, N, K]; out bfloat16 or float32 [tiles * 128, N]. Tiles whose expert is -1 are left alone."""
    _need_cuda(x, w, out, tile_expert)
    lib = load_module("gemm_grouped")
    experts, n, k = w.shape
    tiles = tile_expert.numel()
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
    assert x.shape == (tiles * GROUPED_ROWS, k) and out.shape == (tiles * GROUPED_ROWS, n) and out.stride(1) == 1
    assert out.dtype in (torch.bfloat16, torch.float32)
    _check(lib, lib.abk_gemm_grouped(_p(x), _p(w), _p(out), _ll(out.stride(0)), _i(1 if out.dtype == torch.float32 else 0),
                                     _i(activation), _i(tiles), _i(experts), _i(n), _i(k), _p(tile_expert),
                                     _p(kernel_status(x.device)), _stream()), "gemm_grouped")


def moe_unsort(sorted_out, place, out, n, top, add):
    """out[t] = (out[t] if add else 0) + sum over k of sorted_out[place[t * top + k]], in the order of k; float32."""
    _need_cuda(sorted_out, place, out)
    lib = load_module("gemm_grouped")
    d = out.shape[1]
    assert sorted_out.dtype == out.dtype == torch.float32 and sorted_out.is_contiguous() and out.is_contiguous()
    assert sorted_out.shape[1] == d and place.dtype == torch.int32 and place.numel() >= n * top and out.shape[0] >= n
    _check(lib, lib.abk_moe_unsort(_p(sorted_out), _p(place), _p(out), _i(n), _i(d), _i(top), _i(1 if add else 0), _stream()),
           "moe_unsort")


def columns_norm(src, dst, count, weight, eps, n):
    """dst[t, i] = weight[i] * src[t, i] / sqrt(mean_i(src[t, i]^2) + eps) for i < count, t < n: a run of columns normed
    where it lies in a product's output (rows of any pitch; dst may be src)."""
    _need_cuda(src, dst, weight)
    lib = load_module("latent")
    assert src.dtype == dst.dtype and src.stride(1) == 1 and dst.stride(1) == 1 and src.shape[1] >= count <= dst.shape[1]
    assert weight.dtype == torch.float32 and weight.numel() == count and src.shape[0] >= n and dst.shape[0] >= n
    _check(lib, lib.abk_columns_norm(_p(src), _ll(src.stride(0)), _p(dst), _ll(dst.stride(0)), _i(_dt(src)), _i(n), _i(count),
                                     _p(weight), _f(eps), _stream()), "columns_norm")


# ------------------------------------------------------------------ attention whose values are its keys (csrc/elementwise.cu)
def qkv_prep_whole(src, dst, n_heads, n_kv_heads, head_dim, batch, q_norm, k_norm, eps, cos, sin, rotary_dim, interleaved,
                   cache):
    """Between the q/k product and attention where q and k are each normed over their whole row (q_norm float32
    [heads * head_dim], k_norm [kv heads * head_dim]; None: no norm) and a value head is its key head as projected:
    src rows [q | k | ...] as projected, dst rows [q | k | v] normed, rotated (pairs of the first rotary_dim elements
    of every head) and, for k and v, written to the cache (a cache.LayerKV, or None)."""
    _need_cuda(src, dst, q_norm, k_norm, cos, sin)
    lib = load_module("elementwise")
    n = batch.n_rows
    heads_size = (n_heads + 2 * n_kv_heads) * head_dim
    assert src.dtype == dst.dtype and src.stride(1) == 1 and dst.stride(1) == 1 and src.data_ptr() != dst.data_ptr()
    assert src.shape[1] >= (n_heads + n_kv_heads) * head_dim and dst.shape[1] >= heads_size and min(src.shape[0], dst.shape[0]) >= n
    if cos is not None:
        assert cos.dtype == torch.float32 and cos.shape == sin.shape and cos.shape[1] == rotary_dim // 2
        if batch.max_position >= cos.shape[0]:
            raise KernelError(f"position {batch.max_position} is beyond the rotary table of {cos.shape[0]} positions")
    if q_norm is not None:
        assert q_norm.dtype == k_norm.dtype == torch.float32
        assert q_norm.numel() == n_heads * head_dim and k_norm.numel() == n_kv_heads * head_dim
    if cache is not None:
        assert cache.k.dtype == dst.dtype and cache.k.shape[1:] == (n_kv_heads, cache.tokens_per_page, head_dim)
        assert cache.v.shape == cache.k.shape
    _check(lib, lib.abk_qkv_prep_whole(
        _p(src), _ll(src.stride(0)), _p(dst), _ll(dst.stride(0)), _i(_dt(dst)), _i(n), _i(n_heads), _i(n_kv_heads), _i(head_dim),
        _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(batch.seq_len_after), _p(q_norm), _p(k_norm),
        _f(eps or 0.0), _p(cos), _p(sin), _i(rotary_dim), _i(1 if interleaved else 0),
        _p(cache.k if cache is not None else None), _p(cache.v if cache is not None else None),
        _p(cache.page_table if cache is not None else None), _i(cache.table_width if cache is not None else 0),
        _i(cache.ring_pages if cache is not None else 0), _i(cache.tokens_per_page if cache is not None else 1),
        _i(cache.pinned_pages if cache is not None else 0), _stream()), "qkv_prep_whole")


def gate_heads(x, gate, heads, size, n):
    """x[t, h * size : (h + 1) * size] *= sigmoid(gate[t, h]) for t < n: a gate per head (rows of any pitch)."""
    _need_cuda(x, gate)
    lib = load_module("elementwise")
    assert x.dtype == gate.dtype and x.stride(1) == 1 and gate.stride(1) == 1
    assert x.shape[1] >= heads * size and gate.shape[1] >= heads and x.shape[0] >= n and gate.shape[0] >= n
    _check(lib, lib.abk_gate_heads(_p(x), _ll(x.stride(0)), _p(gate), _ll(gate.stride(0)), _i(_dt(x)), _i(n), _i(heads),
                                   _i(size), _stream()), "gate_heads")


# ------------------------------------------------------------------ the wkv mixer (csrc/wkv.cu)
def token_shift(x, mu, last, out, batch):
    """out[s, t] = x[t] + (x'[t] - x[t]) * mu[s]: the blends of every row with the row before it. x [tokens, d] as
    stored; mu float32 [blends, d]; last float32 [slots, d], the last row each sequence brought in earlier steps (what a
    step's first row of a sequence takes as x'); out [blends, tokens, d] of x's type. A step of one token a sequence also
    leaves the new last rows; a step of prompts does so in a second launch."""
    _need_cuda(x, mu, last, out)
    lib = load_module("wkv")
    n, d = batch.n_rows, x.shape[1]
    blends = mu.shape[0]
    assert x.is_contiguous() and out.is_contiguous() and out.dtype == x.dtype and out.shape[0] == blends and out.shape[2] == d
    assert out.shape[1] >= n and mu.dtype == last.dtype == torch.float32 and mu.is_contiguous() and last.is_contiguous()
    assert mu.shape[1] == d and last.shape[1] == d
    _check(lib, lib.abk_token_shift(_p(x), _i(_dt(x)), _i(n), _i(d), _p(mu), _i(blends), _p(last), _p(out), _ll(out.stride(0)),
                                    _i(1 if batch.is_decode else 0), _p(batch.token_seq), _p(batch.seq_start),
                                    _p(batch.seq_slot), _stream()), "token_shift")
    if not batch.is_decode:
        _check(lib, lib.abk_token_shift_keep(_p(x), _i(_dt(x)), _i(d), _p(last), _p(batch.seq_start), _p(batch.seq_slot),
                                             _i(batch.seq_slot.numel()), _stream()), "token_shift_keep")


def tanh_rows(src, dst, n):
    """dst[:n] = tanh(src[:n]): src float32 or of dst's type, dst float32 or bfloat16, of one shape, rows of any pitch."""
    _need_cuda(src, dst)
    lib = load_module("wkv")
    assert src.stride(1) == 1 and dst.stride(1) == 1 and src.shape[1] == dst.shape[1] and min(src.shape[0], dst.shape[0]) >= n
    _check(lib, lib.abk_tanh_rows(_p(src), _ll(src.stride(0)), _i(_dt(src)), _p(dst), _ll(dst.stride(0)), _i(_dt(dst)), _i(n),
                                  _i(src.shape[1]), _stream()), "tanh_rows")


WKV_SEGMENT = 64        # tokens of a segment of the form for prompts
WKV_SEGMENTS_FROM = 128  # rows of a step (one that is no decode step) from which its sequences are walked in segments


def wkv_scan(proj, r_at, k_at, v_at, n_heads, dim, pre, w0, bonus, state, out, batch, ws=None):
    """The recurrence of a wkv layer for every sequence of the step and every head, float32:
        o = (S + diag(bonus) k v^T)^T r;    S <- diag(exp(-exp(pre + w0))) S + k v^T
    proj [tokens, .] as stored: r, k, v of head h at columns r_at / k_at / v_at + h * dim; pre float32 [tokens, heads * dim];
    w0, bonus float32 [heads * dim]; state float32 [slots, heads, dim, dim] (key, value); out float32 [tokens, heads * dim].
    A decode step, or a small one, walks each sequence token by token. A step of prompts (with ws, a Workspace) walks all
    segments of WKV_SEGMENT tokens at once, twice: for each segment's own sum from an empty state, and, once the states
    between the segments are made from the sums, for the outputs (the same numbers, summed in another order). Which way a
    step goes depends on its rows and sequences alone, not on how long each sequence is."""
    _need_cuda(proj, pre, w0, bonus, state, out)
    lib = load_module("wkv")
    hk = n_heads * dim
    assert proj.stride(1) == 1 and pre.dtype == w0.dtype == bonus.dtype == state.dtype == out.dtype == torch.float32
    assert pre.is_contiguous() and out.is_contiguous() and state.is_contiguous() and pre.shape[1] == out.shape[1] == hk
    assert w0.numel() == bonus.numel() == hk and state.shape[1:] == (n_heads, dim, dim)
    assert proj.shape[1] >= max(r_at, k_at, v_at) + hk
    n_seqs = batch.seq_slot.numel()
    chunk, segments, sums, prods = 0, 0, None, None
    if ws is not None and not batch.is_decode and batch.n_rows >= WKV_SEGMENTS_FROM:
        chunk = WKV_SEGMENT
        segments = -(-batch.n_rows // chunk) + n_seqs  # (at most: every sequence's last segment may be a short one)
        if segments <= 65535:
            sums = ws.get("wkv_sums", (segments, n_heads, dim, dim), torch.float32)
            prods = ws.get("wkv_prods", (segments, n_heads, dim), torch.float32)
        else:
            chunk = segments = 0
    _check(lib, lib.abk_wkv_scan(_p(proj), _ll(proj.stride(0)), _i(_dt(proj)), _i(r_at), _i(k_at), _i(v_at), _i(n_heads), _i(dim),
                                 _p(pre), _p(w0), _p(bonus), _p(state), _p(out), _p(batch.seq_start), _p(batch.seq_slot),
                                 _i(n_seqs), _i(chunk), _i(segments), _p(sums), _p(prods), _stream()), "wkv_scan",
           kernels=3 if chunk else 1)


# ------------------------------------------------------------------ experts by a table (csrc/moe.cu)
def moe_table(batch, table, experts, top, pair_expert, pair_weight, status):
    """pair t * top + k is expert table[token[t], k] with weight 1 / top (table int32 [vocab, top]); rows of padding get -1.
    An entry that names no expert sets bit 0 of status."""
    _need_cuda(table, pair_expert, pair_weight, status)
    lib = load_module("moe")
    n = batch.n_rows
    assert table.dtype == torch.int32 and table.is_contiguous() and table.shape[1] == top
    assert pair_expert.dtype == torch.int32 and pair_weight.dtype == torch.float32 and pair_expert.numel() >= n * top
    _check(lib, lib.abk_moe_table(_p(batch.tokens), _p(batch.token_seq), _p(table), _i(table.shape[0]), _i(experts), _i(top),
                                  _i(n), _p(pair_expert), _p(pair_weight), _p(status), _stream()), "moe_table")


# ------------------------------------------------------------------ a stream made anew before a pass (csrc/streams.cu)
def stream_beside(x, y, x0, out, n):
    """x += y (y None: nothing pending); out[t] = [x[t] | x0[t]] in out's type: the stream beside the embedding, as the
    input of the product that makes the stream anew. x float32 [tokens, 1, d] or [tokens, d], x0 float32 [tokens, d]."""
    _need_cuda(x, y, x0, out)
    lib = load_module("streams")
    d = x0.shape[1]
    assert x.dtype == x0.dtype == torch.float32 and x.is_contiguous() and x0.is_contiguous() and out.is_contiguous()
    assert x.numel() // x.shape[0] == d and out.shape[1] == 2 * d and min(x.shape[0], x0.shape[0], out.shape[0]) >= n
    assert y is None or (y.dtype == torch.float32 and y.is_contiguous() and y.shape[-1] == d and y.shape[0] >= n)
    _check(lib, lib.abk_stream_beside(_p(x), _p(y), _p(x0), _p(out), _i(_dt(out)), _i(n), _i(d), _stream()), "stream_beside")


def add_vector(x, v, n):
    """x[t] += v for t < n (float32; x rows of v's size)."""
    _need_cuda(x, v)
    lib = load_module("streams")
    d = v.numel()
    assert x.dtype == v.dtype == torch.float32 and x.is_contiguous() and v.is_contiguous() and x.numel() // x.shape[0] == d
    _check(lib, lib.abk_add_vector(_p(x), _p(v), _i(n), _i(d), _stream()), "add_vector")
