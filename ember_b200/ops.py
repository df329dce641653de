"""Python face of the CUDA kernels: argument checks, then a ctypes call on the current stream.

There is no CPU fall-back and no library stand-in: every function raises ``KernelError`` if
its tensors are not on a CUDA device or if the compiled library is missing or refuses the
sizes.  Tensors are torch tensors used as typed device buffers.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
EPI_STORE, EPI_STORE_F32, EPI_ADD_F32, EPI_SILU_MUL = 0, 1, 2, 3
EPI_SUMS = 5      # tensor-core product of at most 128 tokens: the fp32 sums stay in the split-K scratch


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dt}")


def _check(t: torch.Tensor, name: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on a CUDA device only (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def _p(t: Optional[torch.Tensor]):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def current_stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


_libs = {}


def _lib(name: str):
    lib = _libs.get(name)
    if lib is None:
        try:
            lib = build.load(name)
        except (build.BuildError, OSError) as e:
            raise KernelError(f"the CUDA kernel library '{name}' is not available: {e}") from e
        _libs[name] = lib
    return lib


_launches = 0


def launch_count() -> int:
    """How many kernel-launching calls this process has made (each launches one or two kernels)."""
    return _launches


def add_launches(n: int) -> None:
    """A replayed CUDA graph launches the kernels that were captured into it."""
    global _launches
    _launches += n


def _call(lib, fn, *args):
    global _launches
    _launches += 1
    rc = fn(*args)
    if rc != 0:
        raise KernelError(lib.ember_last_error().decode("utf-8", "replace"))


# ------------------------------------------------------------------------------ elementwise
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor] = None,
          stream: Optional[int] = None, prev_ids: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """out[t, :] = scale * float(table[tokens[t], :]).  With ``prev_ids`` (int32, device) a token -(r + 1) is
    read as prev_ids[r]: the id the sampler wrote there in the step before."""
    _check(tokens, "tokens", torch.int32)
    if prev_ids is not None:
        _check(prev_ids, "prev_ids", torch.int32)
    _check(table, "table")
    _check(out, "out", torch.float32)
    T, (V, H) = tokens.numel(), table.shape
    if out.shape[-1] != H or out.numel() < T * H:
        raise KernelError(f"embed: output {tuple(out.shape)} does not fit {T} rows of width {H}")
    lib = _lib("elementwise")
    _call(lib, lib.ember_embed, _p(tokens), _p(prev_ids), c_int(prev_ids.numel() if prev_ids is not None else 0),
          _p(table), c_int(dtype_code(table.dtype)), _p(out), c_int(T), c_int(H), c_int(V), c_float(scale), _p(err),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, n_rows: int,
            rows: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """out[r] = weight * x[rows[r] or r] * rsqrt(mean(x^2) + eps); x is fp32, statistics fp32."""
    _check(x, "x", torch.float32)
    _check(weight, "weight", torch.float32)
    _check(out, "out")
    H = x.shape[-1]
    if weight.numel() != H or out.shape[-1] != H or out.numel() < n_rows * H:
        raise KernelError(f"rmsnorm: width {H}, weight {tuple(weight.shape)}, out {tuple(out.shape)} for {n_rows} rows")
    if rows is not None:
        _check(rows, "rows", torch.int32)
    lib = _lib("elementwise")
    _call(lib, lib.ember_rmsnorm, _p(x), _p(rows), _p(weight), c_float(eps), _p(out), c_int(dtype_code(out.dtype)),
          c_int(n_rows), c_int(H), c_void_p(stream if stream is not None else current_stream_ptr()))


def qk_norm_rope_store(qkv: torch.Tensor, T: int, n_heads: int, n_kv: int, head_dim: int,
                       q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                       inv_freq: Optional[torch.Tensor], rotary: int, positions: torch.Tensor, seq_of: torch.Tensor,
                       block_table: torch.Tensor, page: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                       q_out: torch.Tensor, write_kv: bool = True, err: Optional[torch.Tensor] = None,
                       stream: Optional[int] = None) -> None:
    """Per head: optional RMSNorm, rotate-half rotation, q to ``q_out``, k/v into their pages."""
    _check(qkv, "qkv")
    _check(q_out, "q_out", qkv.dtype)
    _check(k_pool, "k_pool", qkv.dtype)
    _check(v_pool, "v_pool", qkv.dtype)
    _check(positions, "positions", torch.int32)
    _check(seq_of, "seq_of", torch.int32)
    _check(block_table, "block_table", torch.int32)
    for w, n in ((q_norm_w, "q_norm_w"), (k_norm_w, "k_norm_w"), (inv_freq, "inv_freq")):
        if w is not None:
            _check(w, n, torch.float32)
    if k_pool.dim() != 4 or k_pool.shape[1] != n_kv or k_pool.shape[2] != page or k_pool.shape[3] != head_dim:
        raise KernelError(f"qk_norm_rope_store: key pool {tuple(k_pool.shape)} is not [pages, {n_kv}, {page}, {head_dim}]")
    if v_pool.shape != k_pool.shape:
        raise KernelError("qk_norm_rope_store: key and value pools differ in shape")
    if inv_freq is not None and inv_freq.numel() * 2 != rotary:
        raise KernelError(f"qk_norm_rope_store: {inv_freq.numel()} frequencies for a rotation of {rotary}")
    lib = _lib("elementwise")
    _call(lib, lib.ember_qk_norm_rope_store, _p(qkv), c_int(dtype_code(qkv.dtype)), c_int(T), c_int(qkv.shape[-1]),
          c_int(n_heads), c_int(n_kv), c_int(head_dim), _p(q_norm_w), _p(k_norm_w), c_float(eps), _p(inv_freq),
          c_int(rotary if inv_freq is not None else 0), _p(positions), _p(seq_of), _p(block_table),
          c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]), _p(q_out), _p(k_pool), _p(v_pool),
          c_int(1 if write_kv else 0), _p(err), c_void_p(stream if stream is not None else current_stream_ptr()))


def qk_norm_rope_store_sums_usable(head_dim: int, rotary: int, width: int) -> bool:
    """Whether the head kernel can take a product's fp32 sums (heads of 128 rotated whole or not at all)."""
    return head_dim == 128 and rotary in (0, 128) and width % 8 == 0


def qk_norm_rope_store_sums(sums: torch.Tensor, T: int, n_heads: int, n_kv: int, q_norm_w: Optional[torch.Tensor],
                            k_norm_w: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor],
                            positions: torch.Tensor, seq_of: torch.Tensor, block_table: torch.Tensor, page: int,
                            k_pool: torch.Tensor, v_pool: torch.Tensor, q_out: torch.Tensor, write_kv: bool = True,
                            err: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """``qk_norm_rope_store`` on the fp32 sums [T, (n_heads + 2 n_kv) * 128] a product left in its scratch
    (``gemm_tc`` with ``EPI_SUMS``): queries and cache are bf16, and every sum read is set back to zero."""
    _check(sums, "sums", torch.float32)
    _check(q_out, "q_out", torch.bfloat16)
    _check(k_pool, "k_pool", torch.bfloat16)
    _check(v_pool, "v_pool", torch.bfloat16)
    _check(positions, "positions", torch.int32)
    _check(seq_of, "seq_of", torch.int32)
    _check(block_table, "block_table", torch.int32)
    for w, n in ((q_norm_w, "q_norm_w"), (k_norm_w, "k_norm_w"), (inv_freq, "inv_freq")):
        if w is not None:
            _check(w, n, torch.float32)
    if sums.dim() != 2 or sums.shape[0] < T or sums.shape[1] != (n_heads + 2 * n_kv) * 128:
        raise KernelError(f"qk_norm_rope_store_sums: sums {tuple(sums.shape)} for {T} tokens and {n_heads}/{n_kv} heads of 128")
    if k_pool.dim() != 4 or tuple(k_pool.shape[1:]) != (n_kv, page, 128) or v_pool.shape != k_pool.shape:
        raise KernelError(f"qk_norm_rope_store_sums: pools {tuple(k_pool.shape)} are not [pages, {n_kv}, {page}, 128]")
    if inv_freq is not None and inv_freq.numel() != 64:
        raise KernelError(f"qk_norm_rope_store_sums: {inv_freq.numel()} frequencies for heads of 128")
    if q_out.numel() < T * n_heads * 128 or positions.numel() < T or seq_of.numel() < T:
        raise KernelError("qk_norm_rope_store_sums: query buffer or token arrays too small")
    lib = _lib("elementwise")
    _call(lib, lib.ember_qk_norm_rope_store_sums, _p(sums), c_int(T), c_int(sums.shape[1]), c_int(n_heads), c_int(n_kv),
          _p(q_norm_w), _p(k_norm_w), c_float(eps), _p(inv_freq), c_int(128 if inv_freq is not None else 0), _p(positions),
          _p(seq_of), _p(block_table), c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]), _p(q_out),
          _p(k_pool), _p(v_pool), c_int(1 if write_kv else 0), _p(err),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def wait_limit_probe(limit_ns: int, err: torch.Tensor, waited_ns: torch.Tensor, stream: Optional[int] = None) -> None:
    """Runs the kernels' bounded barrier wait on a barrier nobody arrives at, with a limit of ``limit_ns`` (at most
    100 ms): the wait gives up, the kernel returns, ``err`` gets the wait-limit bit and ``waited_ns`` (int64[1])
    how long the wait lasted.  For tests of the error path; nothing hangs."""
    _check(err, "err", torch.int32)
    _check(waited_ns, "waited_ns", torch.int64)
    lib = _lib("elementwise")
    _call(lib, lib.ember_wait_limit_probe, ctypes.c_ulonglong(int(limit_ns)), _p(err), _p(waited_ns),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def silu_mul_interleaved(x: torch.Tensor, out: torch.Tensor, n_out: int, stream: Optional[int] = None) -> None:
    _check(x, "x")
    _check(out, "out", x.dtype)
    lib = _lib("elementwise")
    _call(lib, lib.ember_silu_mul_interleaved, _p(x), _p(out), c_int(dtype_code(x.dtype)), c_longlong(n_out),
          c_void_p(stream if stream is not None else current_stream_ptr()))


# ------------------------------------------------------------------------------------ GEMM
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, M: int, epilogue: int = EPI_STORE,
              bias: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """out (+)= a[:M] @ w.T on the fp32 SIMT pipes (true 32-bit when both are float32)."""
    _check(a, "a")
    _check(w, "w")
    _check(out, "out")
    N, K = w.shape
    if a.shape[-1] != K:
        raise KernelError(f"gemm: activations of width {a.shape[-1]} against weights {tuple(w.shape)}")
    n_out = N // 2 if epilogue == EPI_SILU_MUL else N
    want = a.dtype if epilogue in (EPI_STORE, EPI_SILU_MUL) else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm: epilogue {epilogue} writes {want}, the output is {out.dtype}")
    if out.shape[-1] != n_out or out.numel() < M * n_out or a.numel() < M * K:
        raise KernelError(f"gemm: output {tuple(out.shape)} / input {tuple(a.shape)} do not fit M={M} N={n_out}")
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if bias.numel() != N:
            raise KernelError(f"gemm: bias of {bias.numel()} for N={N}")
    lib = _lib("gemm_simt")
    _call(lib, lib.ember_gemm_simt, _p(a), c_int(dtype_code(a.dtype)), c_int(K), _p(w), c_int(dtype_code(w.dtype)),
          c_int(K), _p(bias), _p(out), c_int(n_out), c_int(M), c_int(N), c_int(K), c_int(epilogue),
          c_void_p(stream if stream is not None else current_stream_ptr()))


# ------------------------------------------------------------------------------- attention
ATTENTION_MAX_GROUP = 32     # query heads per key/value head the general attention kernel takes (its ATT_MAX_ROWS)


def attention_tile_queries(group: int) -> int:
    """How many query tokens one tile of the general attention kernel may hold."""
    lib = _lib("attention")
    n = lib.ember_attention_tile_queries(c_int(group))
    if n <= 0:
        raise KernelError(f"attention: {group} query heads per key/value head is more than the kernel takes")
    return n


def attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor, T: int,
              n_heads: int, n_kv: int, head_dim: int, tiles: torch.Tensor, n_tiles: int, tile_q: int,
              block_table: torch.Tensor, page: int, window: int, scale: float, n_splits: int = 1,
              split_keys: int = 0, part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
              err: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """Causal attention of the step's tokens over the paged cache (general SIMT kernel)."""
    _check(q, "q")
    _check(out, "out", q.dtype)
    _check(k_pool, "k_pool", q.dtype)
    _check(v_pool, "v_pool", q.dtype)
    _check(tiles, "tiles", torch.int32)
    _check(block_table, "block_table", torch.int32)
    if k_pool.dim() != 4 or tuple(k_pool.shape[1:]) != (n_kv, page, head_dim) or v_pool.shape != k_pool.shape:
        raise KernelError(f"attention: pools {tuple(k_pool.shape)} are not [pages, {n_kv}, {page}, {head_dim}]")
    if q.numel() < T * n_heads * head_dim or out.numel() < T * n_heads * head_dim:
        raise KernelError("attention: q/out too small for the step")
    if n_splits > 1 and (part_o is not None or part_ml is not None or n_splits > ATTENTION_CLUSTER_SPLITS):
        _check(part_o, "part_o", torch.float32)
        _check(part_ml, "part_ml", torch.float32)
        if part_o.numel() < T * n_heads * n_splits * head_dim or part_ml.numel() < T * n_heads * n_splits * 2:
            raise KernelError("attention: split buffers too small")
    lib = _lib("attention")
    _call(lib, lib.ember_attention, _p(q), _p(k_pool), _p(v_pool), _p(out), c_int(dtype_code(q.dtype)), c_int(T),
          c_int(n_heads), c_int(n_kv), c_int(head_dim), _p(tiles), c_int(n_tiles), c_int(tile_q), _p(block_table),
          c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]), c_int(window), c_float(scale),
          c_int(n_splits), c_int(split_keys), _p(part_o), _p(part_ml), _p(err),
          c_void_p(stream if stream is not None else current_stream_ptr()))


# -------------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor, rows: int,
           stream: Optional[int] = None) -> None:
    """out[r] = token drawn from logits[r] under the packed 32-byte parameter row r."""
    _check(logits, "logits", torch.float32)
    _check(params, "params", torch.uint8)
    _check(out, "out", torch.int32)
    if logits.dim() != 2 or logits.shape[0] < rows or params.numel() < rows * 32 or out.numel() < rows:
        raise KernelError("sample: buffers do not fit the rows")
    lib = _lib("sampling")
    _call(lib, lib.ember_sample, _p(logits), c_int(rows), c_int(logits.shape[1]), _p(params), _p(out),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def argmax(logits: torch.Tensor, out: torch.Tensor, rows: int, part_v: torch.Tensor, part_i: torch.Tensor,
           stream: Optional[int] = None) -> None:
    """out[r] = index of the largest logit of row r, lowest index on ties (greedy sampling)."""
    _check(logits, "logits", torch.float32)
    _check(out, "out", torch.int32)
    _check(part_v, "part_v", torch.float32)
    _check(part_i, "part_i", torch.int32)
    if logits.dim() != 2 or logits.shape[0] < rows or out.numel() < rows or part_v.numel() < rows * 32 or part_i.numel() < rows * 32:
        raise KernelError("argmax: buffers do not fit the rows")
    lib = _lib("sampling")
    _call(lib, lib.ember_argmax, _p(logits), c_int(rows), c_int(logits.shape[1]), _p(part_v), _p(part_i), _p(out),
          c_void_p(stream if stream is not None else current_stream_ptr()))


# ------------------------------------------------------------- tensor-core kernels (bf16)
_tc_scratch = {}
_num_sms = {}
TC_ENABLED = True          # tests switch the tensor-core kernels off to check the general ones alone


def _sms(device) -> int:
    n = _num_sms.get(device)
    if n is None:
        n = torch.cuda.get_device_properties(device).multi_processor_count
        _num_sms[device] = n
    return n


_scratch_version = 0


def scratch_version() -> int:
    """Grows whenever the split-K scratch is (re)allocated: a captured CUDA graph holds the old address and must
    not be replayed afterwards."""
    return _scratch_version


def reserve_scratch(device, floats: int) -> torch.Tensor:
    """Makes the split-K scratch at least ``floats`` long.  A ``Linear`` reserves 128 x its output width when it
    is built, so that a loaded model never grows the scratch inside a step."""
    global _scratch_version
    device = torch.device(device)
    t = _tc_scratch.get(device)
    if t is None or t.numel() < floats:
        t = torch.zeros(max(int(floats), 1 << 20), dtype=torch.float32, device=device)
        _tc_scratch[device] = t
        _scratch_version += 1
    return t


def zero_scratch(device) -> None:
    t = _tc_scratch.get(torch.device(device))
    if t is not None:
        t.zero_()


def _scratch(device, floats: int) -> torch.Tensor:
    """Zero-filled fp32 scratch for split-K partial sums; the kernels leave it zeroed."""
    return reserve_scratch(device, floats)


def gemm_tc_usable(x: torch.Tensor, w: torch.Tensor, bias, epilogue: int) -> bool:
    """Whether the tcgen05 product takes these operands: bf16 activations and weights, no bias,
    K a multiple of 8 (TMA row pitch), an even N for the gated epilogue."""
    if not TC_ENABLED or bias is not None or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    n, k = w.shape
    return k % 8 == 0 and not (epilogue == EPI_SILU_MUL and n % 2)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, M: int, epilogue: int = EPI_STORE,
            err: Optional[torch.Tensor] = None, stream: Optional[int] = None, split_mode: int = 0) -> None:
    """out (+)= a[:M] @ w.T on the tcgen05 tensor cores (bf16 in, fp32 accumulate).  With ``EPI_SUMS`` (``out`` None,
    at most 128 tokens) the fp32 sums are left in the split-K scratch and returned as a view [M, N]: whoever reads
    them sets them back to zero (``qk_norm_rope_store_sums``).
    ``split_mode``: how split-K partial sums are combined (0 automatic, 1 atomics, 2 cluster); 3 runs
    prefill-sized products one tile per block instead of persistently, 4 on pairs of SMs whenever the device
    takes them, 5 never on pairs (for tests and tuning)."""
    _check(a, "a", torch.bfloat16)
    _check(w, "w", torch.bfloat16)
    N, K = w.shape
    if a.shape[-1] != K:
        raise KernelError(f"gemm: activations of width {a.shape[-1]} against weights {tuple(w.shape)}")
    if epilogue == EPI_SUMS:
        if out is not None or not 0 < M <= 128 or a.numel() < M * K:
            raise KernelError(f"gemm: the sums of M={M} tokens stay in the scratch only for 1..128 tokens and without an output")
        scratch = _scratch(a.device, M * N)
        lib = _lib("gemm_tc")
        _call(lib, lib.ember_gemm_tc, _p(a), _p(w), c_void_p(0), c_int(N), c_int(M), c_int(N), c_int(K), c_int(epilogue),
              _p(scratch), c_longlong(scratch.numel()), c_int(_sms(a.device)), c_int(split_mode), _p(err),
              c_void_p(stream if stream is not None else current_stream_ptr()))
        return scratch[:M * N].view(M, N)
    _check(out, "out")
    n_out = N // 2 if epilogue == EPI_SILU_MUL else N
    want = torch.bfloat16 if epilogue in (EPI_STORE, EPI_SILU_MUL) else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm: epilogue {epilogue} writes {want}, the output is {out.dtype}")
    if out.shape[-1] != n_out or out.numel() < M * n_out or a.numel() < M * K:
        raise KernelError(f"gemm: output {tuple(out.shape)} / input {tuple(a.shape)} do not fit M={M} N={n_out}")
    scratch = _scratch(a.device, min(M, 128) * N) if M <= 128 else None
    lib = _lib("gemm_tc")
    _call(lib, lib.ember_gemm_tc, _p(a), _p(w), _p(out), c_int(n_out), c_int(M), c_int(N), c_int(K), c_int(epilogue),
          _p(scratch), c_longlong(scratch.numel() if scratch is not None else 0), c_int(_sms(a.device)), c_int(split_mode),
          _p(err),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def gemm_tc_qkv_usable(x: torch.Tensor, w: torch.Tensor, bias, M: int, n_heads: int, n_kv: int, head_dim: int,
                       rotary: int) -> bool:
    """Whether the fused projection takes this step: bf16, no bias, heads of 128 rotated whole (or not at all),
    more than 128 tokens or at most 16 (the rule of ember_gemm_tc_qkv_supported)."""
    if not gemm_tc_usable(x, w, bias, EPI_STORE):
        return False
    n, k = w.shape
    return (0 < M <= 16 or M > 128) and head_dim == 128 and rotary in (0, 128) and n == (n_heads + 2 * n_kv) * 128


# From how many tokens on a step's q/k/v product finishes the heads itself.  Measured at the 1.7B shape, product +
# head kernel against the fused product: 18.2 / 18.8 us at 256 tokens, 19.7 / 18.8 at 512, 38.2 / 29.3 at 2,048,
# 74.5 / 51.3 at 4,096 (below, the step is one or two tiles an SM and the longer epilogue has no next tile to
# hide behind).
QKV_FUSE_MIN_TOKENS = 512
# Up to how many tokens a decode step's q/k/v product does (product + head kernel against the fused product, in a
# graph: 8.4 / 6.2 us at 1 token, 9.1 / 7.6 at 8, 9.4 / 10.1 at 16: a block of the cluster finishes its share of
# the tokens one after the other, and only the first two are prepared while the product runs).
QKV_FUSE_MAX_DECODE_TOKENS = 8


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, T: int, out: torch.Tensor, stream: Optional[int] = None) -> None:
    """out[i // 2, t] = (cos_i, cos_{i+1}, sin_i, sin_{i+1}) of float(positions[t]) * inv_freq[i] in fp32;
    ``out`` is [frequencies / 2, tokens a row, 4] (token-minor: what the rotating epilogue reads)."""
    _check(positions, "positions", torch.int32)
    _check(inv_freq, "inv_freq", torch.float32)
    _check(out, "out", torch.float32)
    half = inv_freq.numel()
    if out.dim() != 3 or out.shape[0] != half // 2 or out.shape[2] != 4 or out.shape[1] < T or half % 2:
        raise KernelError(f"rope_table: output {tuple(out.shape)} for {half} frequencies and {T} tokens")
    lib = _lib("elementwise")
    _call(lib, lib.ember_rope_table, _p(positions), _p(inv_freq), c_int(T), c_int(half), c_int(out.shape[1]), _p(out),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def gemm_tc_qkv(a: torch.Tensor, w: torch.Tensor, M: int, n_heads: int, n_kv: int, q_norm_w: Optional[torch.Tensor],
                k_norm_w: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor],
                inv_freq: Optional[torch.Tensor], positions: torch.Tensor,
                seq_of: torch.Tensor, block_table: torch.Tensor, page: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                q_out: torch.Tensor, write_kv: bool = True, err: Optional[torch.Tensor] = None,
                stream: Optional[int] = None, split_mode: int = 0) -> None:
    """[q | k | v] = a[:M] @ w.T on the tcgen05 tensor cores with the heads finished in the epilogue: RMSNorm and
    rotation of query and key heads in fp32 on the accumulator, queries to ``q_out``, keys and values into their
    cache pages.  More than 128 tokens rotate with ``cos_sin`` [32, tokens a row, 4] from ``rope_table``, at most
    16 with the frequencies ``inv_freq`` [64] (both None: no rotation).  Heads are 128 wide."""
    _check(a, "a", torch.bfloat16)
    _check(w, "w", torch.bfloat16)
    _check(q_out, "q_out", torch.bfloat16)
    _check(k_pool, "k_pool", torch.bfloat16)
    _check(v_pool, "v_pool", torch.bfloat16)
    _check(positions, "positions", torch.int32)
    _check(seq_of, "seq_of", torch.int32)
    _check(block_table, "block_table", torch.int32)
    for t, n in ((q_norm_w, "q_norm_w"), (k_norm_w, "k_norm_w"), (cos_sin, "cos_sin"), (inv_freq, "inv_freq")):
        if t is not None:
            _check(t, n, torch.float32)
    N, K = w.shape
    if a.shape[-1] != K or a.numel() < M * K:
        raise KernelError(f"gemm_qkv: activations {tuple(a.shape)} against weights {tuple(w.shape)} for M={M}")
    if k_pool.dim() != 4 or tuple(k_pool.shape[1:]) != (n_kv, page, 128) or v_pool.shape != k_pool.shape:
        raise KernelError(f"gemm_qkv: pools {tuple(k_pool.shape)} are not [pages, {n_kv}, {page}, 128]")
    if q_out.numel() < M * n_heads * 128 or positions.numel() < M or seq_of.numel() < M:
        raise KernelError("gemm_qkv: query buffer or token arrays too small")
    if inv_freq is not None and inv_freq.numel() != 64:
        raise KernelError(f"gemm_qkv: {inv_freq.numel()} frequencies for heads of 128")
    if cos_sin is not None and (cos_sin.dim() != 3 or cos_sin.shape[0] != 32 or cos_sin.shape[1] < M or cos_sin.shape[2] != 4):
        raise KernelError(f"gemm_qkv: rotation table {tuple(cos_sin.shape)} is not [32, >= {M}, 4]")
    lib = _lib("gemm_tc")
    _call(lib, lib.ember_gemm_tc_qkv, _p(a), _p(w), c_int(M), c_int(N), c_int(K), c_int(n_heads), c_int(n_kv),
          _p(q_norm_w), _p(k_norm_w), c_float(eps), _p(cos_sin), c_int(cos_sin.shape[1] if cos_sin is not None else 0), _p(inv_freq), _p(positions), _p(seq_of), _p(block_table),
          c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]), _p(q_out), _p(k_pool), _p(v_pool),
          c_int(1 if write_kv else 0), c_int(_sms(a.device)), c_int(split_mode), _p(err),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def num_sms(device) -> int:
    return _sms(device)


def attention_tc_supported(head_dim: int, group: int, page_tokens: int, mode: int) -> bool:
    """Whether the tensor-core attention takes this geometry (mode 0: prompt portions, 1: single tokens)."""
    # the same rule as ember_attention_tc_supported, stated here so that a model that cannot use the
    # kernels never loads (or compiles) their library
    if not TC_ENABLED or head_dim not in (64, 128) or page_tokens not in (16, 32, 64) or group < 1:
        return False
    return group <= 16 if mode == 1 else group <= 64


ATTENTION_CLUSTER_SPLITS = 8     # key splits of a decode tile that one thread-block cluster can merge


def attention_tc_tile_queries(group: int) -> int:
    return 64 // group if 1 <= group <= 64 else 0


FA_ENABLED = True


def attention_fa_supported(head_dim: int, group: int, page_tokens: int) -> bool:
    """Whether the tcgen05 prefill attention takes this geometry (the rule of ember_attention_fa_supported)."""
    return (TC_ENABLED and FA_ENABLED and head_dim == 128 and page_tokens in (16, 32, 64)
            and 1 <= group <= 128 and 128 % group == 0)


def attention_fa_tile_queries(group: int) -> int:
    return 128 // group


def attention_fa(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor, n_heads: int,
                 n_kv: int, head_dim: int, tiles: torch.Tensor, n_tiles: int, block_table: torch.Tensor, page: int,
                 window: int, scale: float, err: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """bf16 causal attention of prompt portions on tcgen05 tensor cores (S and O in tensor memory)."""
    _check(q, "q", torch.bfloat16)
    _check(out, "out", torch.bfloat16)
    _check(k_pool, "k_pool", torch.bfloat16)
    _check(v_pool, "v_pool", torch.bfloat16)
    _check(tiles, "tiles", torch.int32)
    _check(block_table, "block_table", torch.int32)
    if k_pool.dim() != 4 or tuple(k_pool.shape[1:]) != (n_kv, page, head_dim) or v_pool.shape != k_pool.shape:
        raise KernelError(f"attention: pools {tuple(k_pool.shape)} are not [pages, {n_kv}, {page}, {head_dim}]")
    lib = _lib("attention_fa")
    _call(lib, lib.ember_attention_fa, _p(q), _p(k_pool), _p(v_pool), _p(out), c_int(n_heads), c_int(n_kv), c_int(head_dim),
          _p(tiles), c_int(n_tiles), _p(block_table), c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]),
          c_int(window), c_float(scale), _p(err), c_void_p(stream if stream is not None else current_stream_ptr()))


def attention_tc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor, mode: int,
                 n_heads: int, n_kv: int, head_dim: int, tiles: torch.Tensor, n_tiles: int, block_table: torch.Tensor,
                 page: int, window: int, scale: float, n_splits: int = 1, split_keys: int = 0,
                 part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                 err: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """bf16 attention over the paged cache on tensor cores (TMA-fed).  ``mode`` 0 takes tiles of
    prompt portions, 1 takes single-token tiles and may split their key range: with ``part_o`` / ``part_ml`` the
    splits' partial results go through those buffers and a second kernel merges them; without them (at most 8
    splits) the splits of a tile are a thread-block cluster and are merged in shared memory."""
    _check(q, "q", torch.bfloat16)
    _check(out, "out", torch.bfloat16)
    _check(k_pool, "k_pool", torch.bfloat16)
    _check(v_pool, "v_pool", torch.bfloat16)
    _check(tiles, "tiles", torch.int32)
    _check(block_table, "block_table", torch.int32)
    if k_pool.dim() != 4 or tuple(k_pool.shape[1:]) != (n_kv, page, head_dim) or v_pool.shape != k_pool.shape:
        raise KernelError(f"attention: pools {tuple(k_pool.shape)} are not [pages, {n_kv}, {page}, {head_dim}]")
    if n_splits > 1 and (part_o is not None or part_ml is not None or n_splits > ATTENTION_CLUSTER_SPLITS):
        _check(part_o, "part_o", torch.float32)
        _check(part_ml, "part_ml", torch.float32)
        if part_o.numel() < n_tiles * n_heads * n_splits * head_dim or part_ml.numel() < n_tiles * n_heads * n_splits * 2:
            raise KernelError("attention: split buffers too small")
    lib = _lib("attention_tc")
    _call(lib, lib.ember_attention_tc, _p(q), _p(k_pool), _p(v_pool), _p(out), c_int(mode), c_int(n_heads), c_int(n_kv),
          c_int(head_dim), _p(tiles), c_int(n_tiles), _p(block_table), c_int(block_table.shape[-1]), c_int(page),
          c_int(k_pool.shape[0]), c_int(window), c_float(scale), c_int(n_splits), c_int(split_keys), _p(part_o),
          _p(part_ml), _p(err), c_void_p(stream if stream is not None else current_stream_ptr()))
