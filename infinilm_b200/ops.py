"""Python face of the hand-written sm_100a kernels.

Each function checks its arguments on the host (shapes, dtypes, contiguity, device), then calls
the `extern "C"` entry point of the kernel's shared object with raw device pointers and the
current CUDA stream. There is no CPU implementation and no library stand-in here: a tensor that
is not on a CUDA device, or a kernel library that cannot be built, raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


def kind_of(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> _c_void_p:
    if t is None:
        return _c_void_p(0)
    return _c_void_p(t.data_ptr())


_raw_stream = torch._C._cuda_getCurrentRawStream
_cur_device = torch._C._cuda_getDevice


def _stream() -> _c_void_p:
    """The current device's current stream (asked of the runtime directly: this runs once per launch)."""
    return _c_void_p(_raw_stream(_cur_device()))


def _need_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("infinilm_b200 kernels run on a CUDA device only; got a tensor on "
                              f"{t.device} (there is no CPU path)")


def _contig(name: str, t: torch.Tensor) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_launches = 0


def launch_count() -> int:
    """Kernels of this package launched so far (replayed graph nodes included)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(code: int, what: str) -> None:
    global _launches
    if code == 0:
        _launches += 1
        return
    if code == -1:
        raise KernelError(f"{what}: bad argument")
    if code == -2:
        raise KernelError(f"{what}: size not supported by this kernel")
    if code >= 1000:
        raise KernelError(f"{what}: CUDA launch failed (cudaError {code - 1000})")
    raise KernelError(f"{what}: error {code}")


_fns = {}


def _fn(lib_name: str, fn_name: str, argtypes, defines=None):
    """The entry point `fn_name` of the library built from `lib_name` with `defines`; looked up once."""
    key = (lib_name, fn_name, next(iter(defines.values())) if defines else None)
    f = _fns.get(key)
    if f is None:
        if defines and len(defines) != 1:
            raise KernelError("a kernel library is keyed by one definition")
        f = getattr(build.load(lib_name, defines), fn_name)
        f.argtypes = argtypes
        f.restype = _c_int
        _fns[key] = f
    return f


# ----------------------------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor, round_bf16: bool) -> None:
    """out[t,:] (f32) = table[ids[t],:] * scale; rounded through bfloat16 when `round_bf16`."""
    _need_cuda(ids, table, out)
    T, (V, H) = ids.numel(), table.shape
    if ids.dtype != torch.int32 or out.dtype != torch.float32 or out.shape != (T, H):
        raise KernelError("embed: ids int32 [T], out float32 [T,H]")
    _contig("table", table), _contig("out", out)
    f = _fn("embedding", "il_embed", [_c_void_p, _c_void_p, _c_int, _c_float, _c_void_p, _c_int, _c_int,
                                      _c_int, _c_int, _c_void_p])
    _check(f(_ptr(ids), _ptr(table), kind_of(table.dtype), scale, _ptr(out), T, H, V, int(round_bf16),
             _stream()), "embed")


def patch_tokens(token_ids: torch.Tensor, rows: torch.Tensor, src_idx: torch.Tensor, src: torch.Tensor) -> None:
    """token_ids[rows[i]] = src[src_idx[i]], all int32 on the device."""
    _need_cuda(token_ids, rows, src_idx, src)
    for t in (token_ids, rows, src_idx, src):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("patch_tokens: contiguous int32 tensors")
    f = _fn("embedding", "il_patch_tokens", [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p])
    _check(f(_ptr(token_ids), _ptr(rows), _ptr(src_idx), _ptr(src), rows.numel(), _stream()), "patch_tokens")


def add_rmsnorm(resid: torch.Tensor, branch: Optional[torch.Tensor], branch_scale: float, weight: torch.Tensor,
                eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None, vec: Optional[torch.Tensor] = None) -> None:
    """resid += branch_scale * branch (+ vec: float32, one [H] vector for every row or a [T,H] row for each) (f32, in place);
    out = RMSNorm(resid) * weight.

    With `rows` (int32 indices) only those rows are normalised, into out[0..len(rows)), and
    `resid` is left as it was."""
    _need_cuda(resid, branch, weight, out, rows, vec)
    if vec is not None and (vec.dtype != torch.float32 or not vec.is_contiguous()
                            or (vec.numel() != resid.shape[1] and tuple(vec.shape) != tuple(resid.shape))):
        raise KernelError("add_rmsnorm: vec must be a contiguous float32 [H] or [T,H]")
    T, H = resid.shape
    n = T if rows is None else rows.numel()
    if resid.dtype != torch.float32 or weight.numel() != H or out.shape[-1] != H or out.shape[0] < n:
        raise KernelError("add_rmsnorm: resid float32 [T,H], weight [H], out [n,H]")
    if branch is not None and (branch.shape != resid.shape or branch.dtype != out.dtype):
        raise KernelError("add_rmsnorm: branch must match resid's shape and out's dtype")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("add_rmsnorm: rows must be int32")
    _contig("resid", resid), _contig("out", out)
    if branch is not None:
        _contig("branch", branch)
    f = _fn("rmsnorm", "il_add_rmsnorm", [_c_void_p, _c_void_p, _c_float, _c_void_p, _c_int, _c_float, _c_void_p,
                                          _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p])
    _check(f(_ptr(resid), _ptr(branch), branch_scale, _ptr(weight), kind_of(weight.dtype), eps, _ptr(out),
             kind_of(out.dtype), _ptr(rows), n, H, _ptr(vec), H if vec is not None and vec.dim() == 2 else 0, _stream()), "add_rmsnorm")


ACT_SILU, ACT_GELU_TANH = 1, 2                    # the gate of a gated feed-forward


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, act: int = ACT_SILU) -> None:
    """out[t,i] = act(gate_up[t,i]) * gate_up[t,I+i]; act: SiLU or the tanh form of GELU."""
    _need_cuda(gate_up, out)
    T, I2 = gate_up.shape
    if I2 % 2 or out.shape != (T, I2 // 2) or out.dtype != gate_up.dtype:
        raise KernelError("swiglu: gate_up [T,2I], out [T,I] of the same dtype")
    _contig("gate_up", gate_up), _contig("out", out)
    f = _fn("swiglu", "il_swiglu", [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(gate_up), _ptr(out), kind_of(out.dtype), T, I2 // 2, act, _stream()), "swiglu")


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> None:
    _need_cuda(y, bias)
    T, N = y.shape
    if bias.numel() != N:
        raise KernelError("add_bias: bias [N]")
    _contig("y", y)
    f = _fn("swiglu", "il_add_bias", [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(y), kind_of(y.dtype), _ptr(bias), kind_of(bias.dtype), T, N, _stream()), "add_bias")


def rope_store(qkv: torch.Tensor, tok_pos: torch.Tensor, tok_entry: torch.Tensor, block_table: torch.Tensor,
               cache: Optional[torch.Tensor], page_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
               rot_dim: int, inv_freq: Optional[torch.Tensor], mscale: float) -> None:
    """Rotates q and k of `qkv` in place and writes k and v to their cache slots (if `cache`)."""
    _need_cuda(qkv, tok_pos, tok_entry, block_table, cache, inv_freq)
    T = qkv.shape[0]
    _contig("qkv", qkv), _contig("block_table", block_table)
    if tok_pos.dtype != torch.int32 or tok_entry.dtype != torch.int32 or block_table.dtype != torch.int32:
        raise KernelError("rope_store: descriptors must be int32")
    if rot_dim > 0 and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2):
        raise KernelError("rope_store: inv_freq float32 [rot_dim/2]")
    if cache is not None:
        _contig("cache", cache)
        if cache.dtype != qkv.dtype or tuple(cache.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
            raise KernelError("rope_store: cache [pages,2,kv_heads,page,head_dim] of qkv's dtype")
    f = _fn("rope_cache", "il_rope_store", [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                            _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                            _c_float, _c_void_p])
    _check(f(_ptr(qkv), kind_of(qkv.dtype), qkv.shape[1], _ptr(tok_pos), _ptr(tok_entry), _ptr(block_table),
             block_table.shape[1], _ptr(cache), page_size, T, n_heads, n_kv_heads, head_dim, rot_dim,
             _ptr(inv_freq), mscale, _stream()), "rope_store")


def attention_plain(qkv: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                    tok_pos: torch.Tensor, tok_entry: torch.Tensor, page_size: int, n_heads: int,
                    n_kv_heads: int, head_dim: int, scale: float, window: Optional[int] = None,
                    sink: Optional[torch.Tensor] = None, dist_bias: Optional[torch.Tensor] = None) -> None:
    """Causal attention of every token of `qkv` over its request's cache pages (plain kernel). `qkv` needs the query
    heads only (keys and values are read from the cache). `sink`: float32 [heads], a score per head that joins the
    softmax's denominator without a value. `dist_bias`: float32 [far + 1, heads], added to the scaled score of a key n
    positions back as dist_bias[min(n, far), head]."""
    _need_cuda(qkv, out, cache, block_table, tok_pos, tok_entry, sink, dist_bias)
    _check_sink(sink, n_heads)
    _check_dist_bias(dist_bias, n_heads)
    T = qkv.shape[0]
    if out.shape != (T, n_heads * head_dim) or out.dtype != qkv.dtype or cache.dtype != qkv.dtype:
        raise KernelError("attention_plain: out [T, heads*head_dim], same dtype as qkv and cache")
    if head_dim > 1024:
        raise KernelError(f"attention_plain: head_dim {head_dim} > 1024 is not supported")
    _contig("qkv", qkv), _contig("out", out), _contig("cache", cache), _contig("block_table", block_table)
    f = _fn("attn_plain", "il_attn_plain", [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                            _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                                            _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p])
    _check(f(_ptr(qkv), kind_of(qkv.dtype), qkv.shape[1], _ptr(out), _ptr(cache), _ptr(block_table),
             block_table.shape[1], _ptr(tok_pos), _ptr(tok_entry), page_size, T, n_heads, n_kv_heads, head_dim,
             scale, int(window or 0), _ptr(sink), _ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0] - 1, _stream()),
           "attention_plain")


def _check_sink(sink: Optional[torch.Tensor], n_heads: int) -> None:
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != n_heads or not sink.is_contiguous()):
        raise KernelError("attention: sink must be a contiguous float32 tensor, one number per query head")


def _check_dist_bias(dist_bias: Optional[torch.Tensor], n_heads: int) -> None:
    if dist_bias is not None and (dist_bias.dtype != torch.float32 or dist_bias.dim() != 2 or dist_bias.shape[1] != n_heads
                                  or dist_bias.shape[0] < 1 or not dist_bias.is_contiguous()):
        raise KernelError("attention: the distance bias must be a contiguous float32 [far + 1, heads] tensor")


def norm_add(resid: torch.Tensor, branch: torch.Tensor, weight: torch.Tensor, eps: float, scale: float,
             copy: Optional[torch.Tensor] = None) -> None:
    """resid += scale * branch / sqrt(mean(branch^2) + eps) * weight, row by row in float32 (resid float32 [T,H], in place);
    `copy` (of branch's dtype, [T,H]) receives the new rows of resid: what the next sublayer of a model reads whose norms sit
    on the sublayers' outputs."""
    _need_cuda(resid, branch, weight, copy)
    T, H = resid.shape
    if resid.dtype != torch.float32 or tuple(branch.shape) != (T, H) or weight.numel() != H:
        raise KernelError("norm_add: resid float32 [T,H], branch [T,H], weight [H]")
    if copy is not None and (tuple(copy.shape) != (T, H) or copy.dtype != branch.dtype or not copy.is_contiguous()):
        raise KernelError("norm_add: copy [T,H] of the branch's dtype")
    _contig("resid", resid), _contig("branch", branch), _contig("weight", weight)
    f = _fn("rmsnorm", "il_norm_add", [_c_void_p, _c_void_p, _c_float, _c_void_p, _c_int, _c_float, _c_void_p, _c_int, _c_int, _c_int,
                                       _c_void_p])
    _check(f(_ptr(resid), _ptr(branch), scale, _ptr(weight), kind_of(weight.dtype), eps, _ptr(copy), kind_of(branch.dtype), T, H,
             _stream()), "norm_add")


HYPER_MAX_STREAMS = 16


def hyper_step(streams: torch.Tensor, n_streams: int, *, init: Optional[torch.Tensor] = None, y: Optional[torch.Tensor] = None,
               mix: Optional[torch.Tensor] = None, out_w: Optional[torch.Tensor] = None, in_next: Optional[torch.Tensor] = None,
               norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, normed: Optional[torch.Tensor] = None,
               sum_out: Optional[torch.Tensor] = None) -> None:
    """What lies between two sublayers of a model that keeps `n_streams` copies of its residual stream (`streams` float32
    [T, n_streams * H], in place), row by row in float32:
    `init` (float32 [T, H]): every copy starts as this row; `y` [T, H] with `mix` [S, S] and `out_w` [S]: the write-back of the
    sublayer before, x_t <- sum_s mix[s, t] x_s + out_w[t] y; `in_next` [S] with `norm_weight` and `normed` [T, H]: the next
    sublayer's input, RMSNorm(sum_t in_next[t] x_t) * norm_weight; `sum_out` (float32 [T, H]): the sum of the copies."""
    _need_cuda(streams, init, y, mix, out_w, in_next, norm_weight, normed, sum_out)
    T, SH = streams.shape
    S = int(n_streams)
    if streams.dtype != torch.float32 or not streams.is_contiguous() or S < 1 or S > HYPER_MAX_STREAMS or SH % S:
        raise KernelError(f"hyper_step: streams float32 [T, S * H] with 1 <= S <= {HYPER_MAX_STREAMS}")
    H = SH // S
    for name, t in (("init", init), ("sum_out", sum_out)):
        if t is not None and (t.dtype != torch.float32 or tuple(t.shape) != (T, H) or not t.is_contiguous()):
            raise KernelError(f"hyper_step: {name} float32 [T, H]")
    for name, t, n in (("mix", mix, S * S), ("out_w", out_w, S), ("in_next", in_next, S)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
            raise KernelError(f"hyper_step: {name} float32 with {n} entries")
    if y is not None and (mix is None or out_w is None or tuple(y.shape) != (T, H) or not y.is_contiguous()):
        raise KernelError("hyper_step: y [T, H] comes with mix and out_w")
    if in_next is not None and (norm_weight is None or normed is None or norm_weight.numel() != H or tuple(normed.shape) != (T, H)
                                or not normed.is_contiguous()):
        raise KernelError("hyper_step: in_next comes with norm_weight [H] and normed [T, H]")
    if y is not None and normed is not None and y.dtype != normed.dtype:
        raise KernelError("hyper_step: y and normed have one dtype")
    act = y.dtype if y is not None else normed.dtype if normed is not None else torch.float32
    f = _fn("rmsnorm", "il_hyper_step", [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_float,
                                         _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(streams), _ptr(init), _ptr(y), kind_of(act), _ptr(mix), _ptr(out_w), _ptr(in_next), _ptr(norm_weight),
             kind_of(norm_weight.dtype) if norm_weight is not None else 0, eps, _ptr(normed), _ptr(sum_out), S, H, T, _stream()), "hyper_step")


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x rounded to bfloat16; x contiguous float32, out of the same shape."""
    _need_cuda(x, out)
    if x.dtype != torch.float32 or out.dtype != torch.bfloat16 or x.shape != out.shape:
        raise KernelError("cast_rows: float32 in, bfloat16 out, one shape")
    _contig("x", x), _contig("out", out)
    f = _fn("rmsnorm", "il_cast_rows", [_c_void_p, _c_void_p, _c_int, _c_ll, _c_void_p])
    _check(f(_ptr(x), _ptr(out), BF16, x.numel(), _stream()), "cast_rows")


def qk_norm_store(proj: torch.Tensor, q_off: int, k_off: Optional[int], v_off: int, n_heads: int, n_kv_heads: int, qk_dim: int, v_dim: int,
                  head_dim: int, w_q: torch.Tensor, w_k: Optional[torch.Tensor], eps: float, temp_coef: float, temp_every: int,
                  q_out: torch.Tensor, tok_pos: torch.Tensor, tok_entry: torch.Tensor, block_table: torch.Tensor,
                  cache: Optional[torch.Tensor], page_size: int) -> None:
    """Per token and head: q / rms(q) * w_q (times 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1) if temp_every > 0)
    to `q_out` [T, heads * head_dim]; k / rms(k) * w_k to the K plane of the token's cache slot and the value columns (at
    `v_off`; the key columns themselves where the values are the keys as projected) to the V plane. Heads are laid out at
    head_dim >= qk_dim, v_dim, the surplus zero. `k_off` None: the mixer has no keys of its own, only queries are normed."""
    _need_cuda(proj, w_q, w_k, q_out, tok_pos, tok_entry, block_table, cache)
    T = proj.shape[0]
    has_k = k_off is not None
    if proj.stride(1) != 1 or q_off + n_heads * qk_dim > proj.shape[1] or (has_k and (k_off + n_kv_heads * qk_dim > proj.shape[1]
                                                                                    or v_off + n_kv_heads * v_dim > proj.shape[1])):
        raise KernelError("qk_norm_store: segments lie outside the rows")
    if w_q.numel() != qk_dim or (has_k and (w_k is None or w_k.numel() != qk_dim or w_k.dtype != w_q.dtype)):
        raise KernelError("qk_norm_store: one norm weight of qk_dim entries for the queries and one for the keys, of one dtype")
    if tuple(q_out.shape) != (T, n_heads * head_dim) or q_out.dtype != proj.dtype or not q_out.is_contiguous():
        raise KernelError("qk_norm_store: q_out [T, heads * head_dim] of proj's dtype")
    _i32("qk_norm_store", tok_pos, tok_entry, block_table)
    _contig("block_table", block_table)
    if cache is not None:
        _contig("cache", cache)
        if cache.dtype != proj.dtype or tuple(cache.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
            raise KernelError("qk_norm_store: cache [pages,2,kv_heads,page,head_dim] of proj's dtype")
    f = _fn("qk_norm", "il_qk_norm_store", [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                            _c_void_p, _c_void_p, _c_int, _c_float, _c_float, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                            _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(proj), kind_of(proj.dtype), proj.stride(0), q_off, k_off if has_k else -1, v_off, n_heads, n_kv_heads, qk_dim, v_dim,
             head_dim, _ptr(w_q), _ptr(w_k), kind_of(w_q.dtype), eps, temp_coef, temp_every, _ptr(q_out), _ptr(tok_pos), _ptr(tok_entry),
             _ptr(block_table), block_table.shape[1], _ptr(cache if has_k else None), page_size, T, _stream()), "qk_norm_store")


def qk_rows_norm_rope_store(proj: torch.Tensor, q_off: int, k_off: Optional[int], v_off: int, n_heads: int, n_kv_heads: int, qk_dim: int,
                            v_dim: int, head_dim: int, w_q: torch.Tensor, w_k: Optional[torch.Tensor], eps: float, rot_dim: int,
                            inv_freq: Optional[torch.Tensor], q_out: torch.Tensor, tok_pos: torch.Tensor, tok_entry: torch.Tensor,
                            block_table: torch.Tensor, cache: Optional[torch.Tensor], page_size: int) -> None:
    """Per token: all query columns are divided by their common root mean square and multiplied by `w_q` [heads * qk_dim], all
    key columns likewise with `w_k` [kv_heads * qk_dim]; then the first `rot_dim` dimensions of every head turn by
    pos * inv_freq[i] (dimension i paired with i + rot_dim / 2). Queries to `q_out` [T, heads * head_dim], keys and values to
    the K and V plane of the token's cache slot; heads laid out at head_dim, the surplus zero. `k_off` None: queries only."""
    _need_cuda(proj, w_q, w_k, inv_freq, q_out, tok_pos, tok_entry, block_table, cache)
    T = proj.shape[0]
    has_k = k_off is not None
    if proj.stride(1) != 1 or q_off + n_heads * qk_dim > proj.shape[1] or (has_k and (k_off + n_kv_heads * qk_dim > proj.shape[1]
                                                                                    or v_off + n_kv_heads * v_dim > proj.shape[1])):
        raise KernelError("qk_rows_norm_rope_store: segments lie outside the rows")
    if w_q.numel() != n_heads * qk_dim or (has_k and (w_k is None or w_k.numel() != n_kv_heads * qk_dim or w_k.dtype != w_q.dtype)):
        raise KernelError("qk_rows_norm_rope_store: norm weights of heads * qk_dim (queries) and kv_heads * qk_dim (keys) entries, one dtype")
    if rot_dim and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2 or rot_dim % 2 or rot_dim > qk_dim):
        raise KernelError("qk_rows_norm_rope_store: inv_freq float32 [rot_dim / 2], rot_dim even and at most qk_dim")
    if tuple(q_out.shape) != (T, n_heads * head_dim) or q_out.dtype != proj.dtype or not q_out.is_contiguous():
        raise KernelError("qk_rows_norm_rope_store: q_out [T, heads * head_dim] of proj's dtype")
    _i32("qk_rows_norm_rope_store", tok_pos, tok_entry, block_table)
    _contig("block_table", block_table)
    if has_k:
        if cache is None or not cache.is_contiguous() or cache.dtype != proj.dtype or tuple(cache.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
            raise KernelError("qk_rows_norm_rope_store: cache [pages,2,kv_heads,page,head_dim] of proj's dtype")
    f = _fn("qk_norm", "il_qk_rows_norm_rope_store", [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                                      _c_void_p, _c_void_p, _c_int, _c_float, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                                      _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(proj), kind_of(proj.dtype), proj.stride(0), q_off, k_off if has_k else -1, v_off, n_heads, n_kv_heads, qk_dim, v_dim,
             head_dim, _ptr(w_q), _ptr(w_k), kind_of(w_q.dtype), eps, rot_dim, _ptr(inv_freq if rot_dim else None), _ptr(q_out),
             _ptr(tok_pos), _ptr(tok_entry), _ptr(block_table), block_table.shape[1], _ptr(cache if has_k else None), page_size, T,
             _stream()), "qk_rows_norm_rope_store")


def gate_pack(y: torch.Tensor, head_dim: int, gate: Optional[torch.Tensor], g_off: int, out: torch.Tensor, n_heads: int, v_dim: int) -> None:
    """out[t, h*v_dim + c] = y[t, h*head_dim + c] * sigmoid(gate[t, g_off + h*v_dim + c]) for c < v_dim: a gate per output
    column, and heads laid out at head_dim columns come out packed (`gate` None: only that)."""
    _need_cuda(y, gate, out)
    T = y.shape[0]
    if y.dtype != out.dtype or not y.is_contiguous() or not out.is_contiguous():
        raise KernelError("gate_pack: one dtype, contiguous tensors")
    if gate is not None and (gate.dtype != y.dtype or gate.stride(1) != 1 or g_off + n_heads * v_dim > gate.shape[1]):
        raise KernelError("gate_pack: the gate has y's dtype and one column per output column")
    if y.shape[1] != n_heads * head_dim or tuple(out.shape) != (T, n_heads * v_dim):
        raise KernelError("gate_pack: shapes")
    f = _fn("qk_norm", "il_gate_pack", [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(y), kind_of(y.dtype), head_dim, _ptr(gate), 0 if gate is None else gate.stride(0), g_off, _ptr(out), n_heads, v_dim, T,
             _stream()), "gate_pack")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, alpha: float = 1.0,
             bias: Optional[torch.Tensor] = None) -> None:
    """out[M,N] = alpha * a[M,K] @ w[N,K]^T (+ bias), all float32, FP32 pipes only."""
    _need_cuda(a, w, out, bias)
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.float32 or w.dtype != torch.float32 or out.dtype != torch.float32:
        raise KernelError("gemm_f32: float32 tensors")
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_f32: innermost dimension must be contiguous")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_f32: bias float32 [N]")
    f = _fn("gemm_f32", "il_gemm_f32", [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_float,
                                        _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), _ptr(bias), alpha, M, N, K,
             _stream()), "gemm_f32")


_ones_k = {}


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], uniform: Optional[torch.Tensor], out: torch.Tensor, greedy: bool = False) -> None:
    """One token per row of float32 logits [R,V]; per-row temperature, top_k, top_p, uniform number.
    `greedy`: argmax of every row (no parameters needed)."""
    _need_cuda(logits, temperature, top_k, top_p, uniform, out)
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.dtype != torch.int32 or out.numel() < R:
        raise KernelError("sample: logits float32 [R,V] with contiguous rows, out int32 [R]")
    if greedy:
        key = (logits.device, R)
        if key not in _ones_k:
            _ones_k[key] = torch.ones(max(R, 64), dtype=torch.int32, device=logits.device)
        top_k, temperature, top_p, uniform = _ones_k[key], None, None, None
    else:
        for nm, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                          ("top_p", top_p, torch.float32), ("uniform", uniform, torch.float32)):
            if t is None or t.dtype != dt or t.numel() < R or not t.is_contiguous():
                raise KernelError(f"sample: {nm} must be a contiguous {dt} tensor of R entries")
    f = _fn("sampling", "il_sample", [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                      _c_void_p, _c_void_p])
    _check(f(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(uniform),
             _ptr(out), _stream()), "sample")


def attention_decode(qkv: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                     entry_kvlen: torch.Tensor, n_decode: int, page_size: int, n_heads: int, n_kv_heads: int,
                     head_dim: int, scale: float, window: Optional[int], pages_per_split: int, n_splits: int,
                     o_part: torch.Tensor, ml_part: torch.Tensor, kv_map: Optional[torch.Tensor] = None,
                     sink: Optional[torch.Tensor] = None, v_is_k: bool = False, dist_bias: Optional[torch.Tensor] = None) -> None:
    """bfloat16 split-KV attention of token rows [0, n_decode) (entry i = row i, one token each), then the merge of
    the splits (a second launch; with n_splits = 1 there is none and the attention kernel writes `out` itself). A row whose length is 0 gets zeros; a block-table entry below 0 is never followed.
    pages_per_split 0: each request's pages are divided evenly over the n_splits splits.
    kv_map: the cache's tensor map from `kv_tensor_map` (pages then come in by TMA tensor copies).
    v_is_k: the caller vouches that the V plane of every page repeats its K plane (a latent that is key and value at once);
    with a tensor map only the K plane is then read, half the bytes.
    Scratch: o_part float32 [n_decode*heads*n_splits*head_dim], ml_part float32 [n_decode*heads*n_splits*2]."""
    _need_cuda(qkv, out, cache, block_table, entry_kvlen, o_part, ml_part, sink, dist_bias)
    _check_sink(sink, n_heads)
    _check_dist_bias(dist_bias, n_heads)      # float32 [far + 1, heads]: added to the scaled score of a key n positions back
    if qkv.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_decode: bfloat16 tensors")
    if o_part is None or ml_part is None or o_part.dtype != torch.float32 or ml_part.dtype != torch.float32:
        raise KernelError("attention_decode: scratch must be float32")
    need = n_decode * n_heads * n_splits
    if o_part.numel() < need * head_dim or ml_part.numel() < need * 2:
        raise KernelError("attention_decode: scratch too small")
    if out.shape[1] != n_heads * head_dim or out.shape[0] < n_decode or qkv.shape[0] < n_decode:
        raise KernelError("attention_decode: out [rows, heads*head_dim]")
    if block_table.dtype != torch.int32 or entry_kvlen.dtype != torch.int32 or block_table.shape[0] < n_decode or entry_kvlen.numel() < n_decode:
        raise KernelError("attention_decode: block_table int32 [entries, width], entry_kvlen int32 [entries]")
    _contig("qkv", qkv), _contig("out", out), _contig("cache", cache), _contig("block_table", block_table)
    f = _fn("attn_decode", "il_attn_decode", [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int,
                                              _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_void_p,
                                              _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p],
            defines={"HEAD_DIM": head_dim})
    if kv_map is not None and (kv_map.is_cuda or kv_map.dtype != torch.uint8 or kv_map.numel() != KV_MAP_BYTES):
        raise KernelError("attention_decode: kv_map must be the host tensor kv_tensor_map returned")
    _check(f(_ptr(qkv), qkv.shape[1], _ptr(out), _ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(entry_kvlen),
             page_size, n_decode, n_heads, n_kv_heads, head_dim, scale, int(window or 0), pages_per_split, n_splits,
             _ptr(o_part), _ptr(ml_part), _ptr(kv_map), _ptr(stream_status(qkv.device)) if kv_map is not None else _c_void_p(0),
             _ptr(sink), 1 if v_is_k else 0, _ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0] - 1, _stream()), "attention_decode")
    if n_splits > 1:
        count_launches(1)                         # the merge kernel (a single split needs none: the attention kernel finishes the rows)


_resident = {}


def attention_decode_resident_blocks(head_dim: int, v_is_k: bool = False) -> int:
    """Blocks of the decode attention kernel that the current device runs at once at this head size (occupancy x SMs);
    `v_is_k`: in the form that stages the K plane alone."""
    key = (torch.cuda.current_device(), head_dim, bool(v_is_k))
    if key not in _resident:
        lib = build.load("attn_decode", {"HEAD_DIM": head_dim})
        fn = lib.il_attn_decode_resident_blocks_shared if v_is_k else lib.il_attn_decode_resident_blocks
        fn.argtypes, fn.restype = [], _c_int
        n = int(fn())
        if n <= 0:
            raise KernelError("attention_decode: the occupancy query failed")
        _resident[key] = n
    return _resident[key]


KV_MAP_BYTES = 512


def kv_tensor_map(cache: torch.Tensor) -> Optional[torch.Tensor]:
    """The TMA tensor maps (4 x 128 bytes, on the host) of one layer's bfloat16 cache [pages,2,kv_heads,16,head_dim]: one
    for boxes of [16 keys x 64 columns], one whose box is a whole page of a kv head, one whose box is the K or V of a page
    as tensor-core tiles, one whose box is the K plane of a page (the last three all zero if the driver refuses them).
    None when the attention kernels have no tensor-copy path for this geometry (head_dim not a multiple of 64, or beyond 256)."""
    if (not cache.is_cuda or cache.dtype != torch.bfloat16 or cache.dim() != 5 or cache.shape[3] != 16 or cache.shape[4] % 64
            or cache.shape[4] > 256):
        return None
    hd = cache.shape[4]
    lib = build.load("attn_decode", {"HEAD_DIM": hd})
    fn = lib.il_attn_decode_kv_map
    fn.argtypes, fn.restype = [_c_void_p, _c_void_p, ctypes.c_longlong, _c_int, _c_int], _c_int
    m = torch.zeros(KV_MAP_BYTES, dtype=torch.uint8)
    rc = fn(_c_void_p(m.data_ptr()), _ptr(cache), cache.numel() // hd, hd, cache.shape[2])
    return m if rc == 0 else None


def attention_prefill(qkv: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                      entry_qstart: torch.Tensor, entry_kvlen: torch.Tensor, first_entry: int, n_entries: int,
                      n_tiles_total: int, page_size: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                      window: Optional[int], sink: Optional[torch.Tensor] = None, dist_bias: Optional[torch.Tensor] = None) -> None:
    """bfloat16 causal attention of the tokens of entries [first_entry, n_entries) over their cache pages.
    n_tiles_total = sum over those entries of ceil(q_len / (64 // (heads/kv_heads)))."""
    _need_cuda(qkv, out, cache, block_table, entry_qstart, entry_kvlen, sink, dist_bias)
    _check_sink(sink, n_heads)
    _check_dist_bias(dist_bias, n_heads)
    if qkv.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_prefill: bfloat16 tensors")
    if out.shape != (qkv.shape[0], n_heads * head_dim):
        raise KernelError("attention_prefill: out [T, heads*head_dim]")
    _contig("qkv", qkv), _contig("out", out), _contig("cache", cache), _contig("block_table", block_table)
    f = _fn("attn_prefill", "il_attn_prefill", [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
                                                _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                                                _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p], defines={"HEAD_DIM": head_dim})
    _check(f(_ptr(qkv), qkv.shape[1], _ptr(out), _ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(entry_qstart),
             _ptr(entry_kvlen), page_size, first_entry, n_entries, n_tiles_total, n_heads, n_kv_heads, head_dim, scale,
             int(window or 0), _ptr(sink), _ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0] - 1, _stream()), "attention_prefill")


_tc5_prefill_rows = {}


def prefill_tc5_rows(head_dim: int) -> int:
    """Rows (tokens x heads of a kv head) a block of the tensor-memory prefill kernel owns."""
    if head_dim not in _tc5_prefill_rows:
        lib = build.load("attn_prefill_tc5", {"HEAD_DIM": head_dim})
        fn = lib.il_attn_prefill_tc5_rows
        fn.argtypes, fn.restype = [], _c_int
        _tc5_prefill_rows[head_dim] = int(fn())
    return _tc5_prefill_rows[head_dim]


def prefill_tc5_ok(head_dim: int, group: int, page_size: int, kv_map: Optional[torch.Tensor] = None) -> bool:
    """Whether the tensor-memory prefill kernel takes this geometry and, if given, this tensor map of the cache (it
    needs the third map of `kv_tensor_map`, a page's K or V as tensor-core tiles)."""
    if not (head_dim in (64, 128, 256) and 0 < group <= 128 and page_size == 16):
        return False
    return kv_map is None or _has_third_map(kv_map)


def _has_third_map(kv_map: torch.Tensor) -> bool:
    """Whether this host tensor is a `kv_tensor_map` result with its third map filled; looked at once per tensor
    object (the answer is kept on the object, so another tensor at the same address is looked at again)."""
    ok = getattr(kv_map, "_il_third_map", None)
    if ok is None:
        ok = (not kv_map.is_cuda and kv_map.dtype == torch.uint8 and kv_map.numel() == KV_MAP_BYTES
              and bool(kv_map[256:384].any()))
        kv_map._il_third_map = ok
    return ok


def attention_prefill_tc5(qkv: torch.Tensor, out: torch.Tensor, kv_map: torch.Tensor, block_table: torch.Tensor,
                          entry_qstart: torch.Tensor, entry_kvlen: torch.Tensor, first_entry: int, n_entries: int,
                          n_tiles_total: int, page_size: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                          window: Optional[int], sink: Optional[torch.Tensor] = None, dist_bias: Optional[torch.Tensor] = None) -> None:
    """The same attention as `attention_prefill`, on tcgen05 tensor cores with tensor memory; `kv_map` is the cache's
    tensor map (`kv_tensor_map`). n_tiles_total = sum over the entries of ceil(q_len / (prefill_tc5_rows(head_dim) // (heads/kv_heads)))."""
    _need_cuda(qkv, out, block_table, entry_qstart, entry_kvlen, sink, dist_bias)
    _check_sink(sink, n_heads)
    _check_dist_bias(dist_bias, n_heads)
    if qkv.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc5: bfloat16 tensors")
    if not _has_third_map(kv_map):
        raise KernelError("attention_prefill_tc5: kv_map must be the host tensor kv_tensor_map returned, with its third map")
    if out.shape != (qkv.shape[0], n_heads * head_dim):
        raise KernelError("attention_prefill_tc5: out [T, heads*head_dim]")
    _contig("qkv", qkv), _contig("out", out), _contig("block_table", block_table)
    f = _fn("attn_prefill_tc5", "il_attn_prefill_tc5",
            [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_float, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p], defines={"HEAD_DIM": head_dim})
    _check(f(_ptr(qkv), qkv.shape[1], _ptr(out), _c_void_p(kv_map.data_ptr() + 256), _ptr(block_table), block_table.shape[1],
             _ptr(entry_qstart), _ptr(entry_kvlen), page_size, first_entry, n_entries, n_tiles_total, n_heads, n_kv_heads,
             head_dim, scale, int(window or 0), _ptr(stream_status(qkv.device)), _ptr(sink), _ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0] - 1,
             _stream()), "attention_prefill_tc5")


SKINNY_MAX_ROWS = 16


class ResidualCopy:
    """What a block hands to the next when nothing is pending: the residual stream is complete, and `rows` holds it in the
    compute dtype (the float32 stream itself on the 32-bit path) for a sublayer that reads the stream as it is."""
    __slots__ = ("rows",)

    def __init__(self, rows: torch.Tensor):
        self.rows = rows


class StreamSet:
    """What a block of a model with several copies of its residual stream hands the next one: the copies (float32
    [T, S * H], all write-backs done) and, if the block prepared it, the next block's first normed input. Nothing is pending;
    the model's `resid` holds the copies' sum whenever `normed` is None."""
    __slots__ = ("streams", "n_streams", "normed")
    nothing_pending = True

    def __init__(self, streams: torch.Tensor, n_streams: int, normed: Optional[torch.Tensor] = None):
        self.streams, self.n_streams, self.normed = streams, n_streams, normed


class NormedInput:
    """Activations whose RMSNorm is not finished: `xw` = residual * norm weight (bfloat16 [T,H]) and `sumsq`, the sums of
    the residual's squares per row and block of 16 columns (float32 [T, n_blocks]); the product that reads them divides
    by the rms. Made by `gemm_skinny_resid`, read by `gemm_skinny(glu=True)` and `gemm_skinny_rope`."""
    __slots__ = ("xw", "sumsq", "width", "eps")

    def __init__(self, xw: torch.Tensor, sumsq: torch.Tensor, width: int, eps: float):
        self.xw, self.sumsq, self.width, self.eps = xw, sumsq, int(width), float(eps)

    @property
    def shape(self):
        return self.xw.shape


NORM_MAX_BLOCKS = 256                             # blocks of 16 columns the fused norm handles: residual width <= 4096


def _norm_args(norm_in: Optional[NormedInput], M: int):
    if norm_in is None:
        return _c_void_p(0), 0, 0, 0.0
    sq = norm_in.sumsq
    if sq.dtype != torch.float32 or not sq.is_contiguous() or sq.shape[0] < M or sq.shape[1] > NORM_MAX_BLOCKS:
        raise KernelError("norm_in: sumsq float32 [rows, blocks <= 256], contiguous")
    return _ptr(sq), sq.shape[1], norm_in.width, norm_in.eps


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, alpha: float = 1.0,
                bias: Optional[torch.Tensor] = None, glu: int = 0, norm_in: Optional[NormedInput] = None) -> None:
    """out[M,N] = alpha * x[M,K] @ w[N,K]^T (+ bias) for M <= 16 bfloat16 rows; out bfloat16 or float32.
    glu (True, or ACT_SILU / ACT_GELU_TANH): w is [2N,K] (gate rows, then up rows) and out[M,N] = act(gate) * up.
    norm_in: x is `norm_in.xw`, and the results are divided by the rms that its sums give."""
    _need_cuda(x, w, out, bias)
    M, K = x.shape
    N = w.shape[0] // 2 if glu else w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_skinny: bfloat16 x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_skinny: innermost dimension must be contiguous")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != w.shape[0]):
        raise KernelError("gemm_skinny: bias float32, one per weight row")
    f = _fn("gemm_skinny", "il_gemm_skinny", [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p,
                                              _c_float, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_float,
                                              _c_void_p])
    np_, nb, nw, ne = _norm_args(norm_in, M)
    _check(f(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), kind_of(out.dtype), out.stride(0), _ptr(bias), alpha,
             M, N, K, int(glu), np_, nb, nw, ne, _stream()), "gemm_skinny")


def skinny_resid_ok(M: int, K: int, width: int) -> bool:
    """Whether `gemm_skinny_resid` takes this shape."""
    return 0 < M <= SKINNY_MAX_ROWS and K % 8 == 0 and (width + 15) // 16 <= NORM_MAX_BLOCKS


def gemm_skinny_resid(x: torch.Tensor, w: torch.Tensor, alpha: float, bias: Optional[torch.Tensor], resid: torch.Tensor,
                      branch_scale: float, norm_weight: torch.Tensor, eps: float, xw: torch.Tensor,
                      sumsq: torch.Tensor) -> NormedInput:
    """The last product of a branch (up to 16 bfloat16 rows) with the residual add and the next RMSNorm's inputs in its
    epilogue: resid (float32 [M,H], in place) += branch_scale * bf16(alpha * x @ w^T + bias); xw = resid * norm_weight;
    sumsq[m][b] = sum of resid[m]^2 over columns 16b..16b+15. Returns what the next product needs to finish the norm."""
    _need_cuda(x, w, bias, resid, norm_weight, xw, sumsq)
    M, K = x.shape
    H = w.shape[0]
    nb = (H + 15) // 16
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError(f"gemm_skinny_resid: bfloat16 x{tuple(x.shape)} w{tuple(w.shape)}")
    if resid.dtype != torch.float32 or tuple(resid.shape) != (M, H) or xw.dtype != torch.bfloat16 or tuple(xw.shape) != (M, H):
        raise KernelError("gemm_skinny_resid: resid float32 [M,H], xw bfloat16 [M,H]")
    if sumsq.dtype != torch.float32 or tuple(sumsq.shape) != (M, nb) or norm_weight.numel() != H:
        raise KernelError("gemm_skinny_resid: sumsq float32 [M, ceil(H/16)], norm_weight [H]")
    if x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm_skinny_resid: innermost dimension must be contiguous")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != H):
        raise KernelError("gemm_skinny_resid: bias float32 [H]")
    _contig("resid", resid), _contig("xw", xw), _contig("sumsq", sumsq), _contig("norm_weight", norm_weight)
    f = _fn("gemm_skinny", "il_gemm_skinny_resid", [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_float, _c_int, _c_int, _c_int,
                                                    _c_void_p, _c_float, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias), alpha, M, H, K, _ptr(resid), branch_scale, _ptr(norm_weight),
             kind_of(norm_weight.dtype), _ptr(xw), _ptr(sumsq), _stream()), "gemm_skinny_resid")
    return NormedInput(xw, sumsq, H, eps)


def skinny_rope_ok(M: int, K: int, head_dim: int, rot_dim: int) -> bool:
    """Whether `gemm_skinny_rope` takes this shape: a few rows, rotary and head sizes in steps of 16."""
    return 0 < M <= SKINNY_MAX_ROWS and K % 8 == 0 and head_dim % 16 == 0 and rot_dim % 16 == 0 and 0 <= rot_dim <= head_dim


def gemm_skinny_rope(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, alpha: float, bias: Optional[torch.Tensor],
                     tok_pos: torch.Tensor, tok_entry: torch.Tensor, block_table: torch.Tensor, cache: Optional[torch.Tensor],
                     page_size: int, n_heads: int, n_kv_heads: int, head_dim: int, rot_dim: int,
                     inv_freq: Optional[torch.Tensor], mscale: float, norm_in: Optional[NormedInput] = None) -> None:
    """The q/k/v projection of up to 16 bfloat16 rows with what `rope_store` does in its epilogue: out[M, (heads + 2
    kv_heads) * head_dim] = alpha * x @ w^T (+ bias), q and k rotated, k and v written to their cache slots (if `cache`)."""
    _need_cuda(x, w, out, bias, tok_pos, tok_entry, block_table, cache, inv_freq)
    M, K = x.shape
    N = (n_heads + 2 * n_kv_heads) * head_dim
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or tuple(w.shape) != (N, K) or out.shape != (M, N):
        raise KernelError(f"gemm_skinny_rope: bfloat16 x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_skinny_rope: innermost dimension must be contiguous")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_skinny_rope: bias float32, one per weight row")
    if tok_pos.dtype != torch.int32 or tok_entry.dtype != torch.int32 or block_table.dtype != torch.int32 or tok_pos.numel() < M:
        raise KernelError("gemm_skinny_rope: descriptors must be int32, one position and entry per row")
    if rot_dim > 0 and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2):
        raise KernelError("gemm_skinny_rope: inv_freq float32 [rot_dim/2]")
    _contig("block_table", block_table)
    if cache is not None:
        _contig("cache", cache)
        if cache.dtype != torch.bfloat16 or tuple(cache.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
            raise KernelError("gemm_skinny_rope: cache bfloat16 [pages,2,kv_heads,page,head_dim]")
    f = _fn("gemm_skinny", "il_gemm_skinny_rope",
            [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_float, _c_int, _c_int, _c_void_p, _c_void_p,
             _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_float, _c_void_p, _c_int, _c_int,
             _c_float, _c_void_p])
    np_, nb, nw, ne = _norm_args(norm_in, M)
    _check(f(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), _ptr(bias), alpha, M, K, _ptr(tok_pos),
             _ptr(tok_entry), _ptr(block_table), block_table.shape[1], _ptr(cache), page_size, n_heads, n_kv_heads, head_dim,
             rot_dim, _ptr(inv_freq), mscale, np_, nb, nw, ne, _stream()), "gemm_skinny_rope")


def skinny_ok(M: int, K: int) -> bool:
    return 0 < M <= SKINNY_MAX_ROWS and K % 8 == 0


_stream_status = {}


def stream_status(device) -> torch.Tensor:
    """The status word of the bulk-copy kernels on `device`: 0, or non-zero after a bounded wait ran out."""
    key = torch.device(device).index or 0
    if key not in _stream_status:
        _stream_status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _stream_status[key]


def check_status(device) -> None:
    """Raises if a kernel with bounded waits (mbarriers of the TMA / tcgen05 kernels) gave up since the last check: its
    output is then not to be trusted. Reads one word from the device, so it synchronises; call it where the host
    waits anyway."""
    key = torch.device(device).index or 0
    t = _stream_status.get(key)
    if t is None:
        return
    code = int(t.item())
    if code:
        t.zero_()
        raise KernelError(f"a kernel's bounded wait ran out (code {code}: 11-14 gemm_tc5, 21 attn_decode, 30-39 attn_prefill_tc5, 51-54 gemm_mid); the step's results are invalid")


TC5_MAX_ROWS = 256


def gemm_tc5(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, alpha: float = 1.0, bias: Optional[torch.Tensor] = None,
             scratch: Optional[torch.Tensor] = None) -> None:
    """out[M,N] = alpha * x[M,K] @ w[N,K]^T (+ bias) on the tcgen05 tensor cores (TMA-fed, accumulators in TMEM),
    M <= 256, bfloat16 inputs, out bfloat16 or float32. `scratch`: float32 buffer of `gemm_tc5_scratch_bytes` bytes
    (needed when the kernel slices K to fill the SMs)."""
    _need_cuda(x, w, out, bias, scratch)
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_tc5: bfloat16 x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_tc5: innermost dimension must be contiguous")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tc5: bias float32 [N]")
    need = gemm_tc5_scratch_bytes(M, N, K)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() * 4 < need):
        raise KernelError(f"gemm_tc5: needs {need} bytes of float32 scratch")
    f = _fn("gemm_tc5", "il_gemm_tc5", [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_float,
                                        _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), kind_of(out.dtype), out.stride(0), _ptr(bias), alpha,
             M, N, K, _ptr(scratch), _ptr(stream_status(x.device)), _stream()), "gemm_tc5")


def gemm_tc5_scratch_bytes(M: int, N: int, K: int) -> int:
    lib = build.load("gemm_tc5")
    fn = lib.il_gemm_tc5_scratch_bytes
    fn.argtypes, fn.restype = [_c_int, _c_int, _c_int], ctypes.c_longlong
    return int(fn(M, N, K))


def tc5_ok(M: int, K: int) -> bool:
    return SKINNY_MAX_ROWS < M <= TC5_MAX_ROWS and K % 8 == 0



MID_MAX_ROWS = 128


def mid_ok(M: int, K: int) -> bool:
    return SKINNY_MAX_ROWS < M <= MID_MAX_ROWS and K % 8 == 0


def gemm_mid(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, alpha: float = 1.0, bias: Optional[torch.Tensor] = None,
             glu: int = 0, nb: int = 0, bm: int = 0) -> None:
    """out[M,N] = alpha * x[M,K] @ w[N,K]^T (+ bias) for 17..128 bfloat16 rows on the tcgen05 tensor cores: tiles of 64
    or 128 weight rows (`bm`; the A operand) by blocks of `nb` activation rows (0: chosen by the kernel) over all of K; out bfloat16
    or float32. glu (True, or ACT_SILU / ACT_GELU_TANH): w is [2N,K] (gate rows, then up rows) and out[M,N] = act(gate) * up (bfloat16)."""
    _need_cuda(x, w, out, bias)
    M, K = x.shape
    N = w.shape[0] // 2 if glu else w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_mid: bfloat16 x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_mid: innermost dimension must be contiguous")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != w.shape[0]):
        raise KernelError("gemm_mid: bias float32, one per weight row")
    f = _fn("gemm_mid", "il_gemm_mid", [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_float,
                                        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), kind_of(out.dtype), out.stride(0), _ptr(bias), alpha,
             M, N, K, int(glu), nb, bm, _ptr(stream_status(x.device)), _stream()), "gemm_mid")


_c_ll = ctypes.c_longlong


def embed_pair_pos(ids: torch.Tensor, tok_pos: torch.Tensor, tok_entry: torch.Tensor, entry_qstart: torch.Tensor, table: torch.Tensor,
                   scale: float, pair_table: Optional[torch.Tensor], buckets: int, mul_prev: int, mul_cur: int,
                   prev_state: Optional[torch.Tensor], read_slots: Optional[torch.Tensor], write_slots: Optional[torch.Tensor],
                   inv_freq: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[t,:] (f32) = table[ids[t]] * scale + pair_table[(prev * mul_prev + ids[t] * mul_cur) mod buckets] (row `buckets`
    at position 0) + sinusoid(tok_pos[t]) (entry 2i: sin(pos * inv_freq[i]), 2i+1: cos). The previous token of an entry's
    first token is `prev_state[read_slots[entry]] - 1`; the entry's last token + 1 goes to `prev_state[write_slots[entry]]`."""
    _need_cuda(ids, tok_pos, tok_entry, entry_qstart, table, pair_table, prev_state, read_slots, write_slots, inv_freq, out)
    T, (V, H) = ids.numel(), table.shape
    if out.dtype != torch.float32 or out.shape != (T, H):
        raise KernelError("embed_pair_pos: out float32 [T,H]")
    for t in (ids, tok_pos, tok_entry, entry_qstart, prev_state, read_slots, write_slots):
        if t is not None and t.dtype != torch.int32:
            raise KernelError("embed_pair_pos: descriptors and the state are int32")
    if pair_table is not None and (pair_table.dtype != table.dtype or tuple(pair_table.shape) != (buckets + 1, H)):
        raise KernelError("embed_pair_pos: pair_table [buckets + 1, H] of the table's dtype")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != (H + 1) // 2):
        raise KernelError("embed_pair_pos: inv_freq float32 [ceil(H/2)]")
    _contig("table", table), _contig("out", out)
    if pair_table is not None:
        _contig("pair_table", pair_table)
    f = _fn("embedding", "il_embed_pair_pos", [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_float, _c_void_p, _c_int,
                                               _c_ll, _c_ll, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                                               _c_int, _c_void_p])
    _check(f(_ptr(ids), _ptr(tok_pos), _ptr(tok_entry), _ptr(entry_qstart), _ptr(table), kind_of(table.dtype), scale, _ptr(pair_table),
             int(buckets), int(mul_prev), int(mul_cur), _ptr(prev_state), _ptr(read_slots), _ptr(write_slots), _ptr(inv_freq),
             _ptr(out), T, H, V, _stream()), "embed_pair_pos")


def latent_norm_store(proj: torch.Tensor, off_a: int, n_a: int, off_b: int, n_b: int, w_a: Optional[torch.Tensor],
                      w_b: torch.Tensor, eps: float, out_a: Optional[torch.Tensor], out_b: Optional[torch.Tensor],
                      tok_pos: torch.Tensor, tok_entry: torch.Tensor, block_table: torch.Tensor, cache: Optional[torch.Tensor],
                      page_size: int) -> None:
    """Per row of `proj`: columns [off_a, off_a + n_a) and [off_b, off_b + n_b) are each divided by their root mean
    square (f32) and multiplied by `w_a` / `w_b`. The first goes to `out_a` [T, n_a]; the second to `out_b` (if given) and
    into the token's slot of `cache` [pages, 2, 1, page, n_b], K plane and V plane alike."""
    _need_cuda(proj, w_a, w_b, out_a, out_b, tok_pos, tok_entry, block_table, cache)
    T = proj.shape[0]
    if proj.stride(1) != 1 or off_a + n_a > proj.shape[1] or off_b + n_b > proj.shape[1]:
        raise KernelError("latent_norm_store: segments lie outside the rows")
    if n_a and (w_a is None or w_a.numel() != n_a or out_a is None or tuple(out_a.shape) != (T, n_a) or out_a.dtype != proj.dtype):
        raise KernelError("latent_norm_store: w_a [n_a], out_a [T, n_a] of proj's dtype")
    if w_b.numel() != n_b or (n_a and w_a.dtype != w_b.dtype):
        raise KernelError("latent_norm_store: w_b [n_b], of w_a's dtype")
    if out_b is not None and (tuple(out_b.shape) != (T, n_b) or out_b.dtype != proj.dtype or not out_b.is_contiguous()):
        raise KernelError("latent_norm_store: out_b [T, n_b] of proj's dtype")
    if tok_pos.dtype != torch.int32 or tok_entry.dtype != torch.int32 or block_table.dtype != torch.int32:
        raise KernelError("latent_norm_store: descriptors must be int32")
    _contig("block_table", block_table)
    if cache is not None:
        _contig("cache", cache)
        if cache.dtype != proj.dtype or tuple(cache.shape[1:]) != (2, 1, page_size, n_b):
            raise KernelError("latent_norm_store: cache [pages,2,1,page,n_b] of proj's dtype")
    f = _fn("latent", "il_latent_norm_store", [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int,
                                               _c_float, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int,
                                               _c_int, _c_void_p])
    _check(f(_ptr(proj), kind_of(proj.dtype), proj.stride(0), off_a, n_a, off_b, n_b, _ptr(w_a), _ptr(w_b), kind_of(w_b.dtype), eps,
             _ptr(out_a), _ptr(out_b), _ptr(tok_pos), _ptr(tok_entry), _ptr(block_table), block_table.shape[1], _ptr(cache), page_size,
             T, _stream()), "latent_norm_store")


def sigmoid_gate(y: torch.Tensor, gate: torch.Tensor) -> None:
    """y[t, :] *= sigmoid(gate[t, :]) in place; y [T, n] contiguous, gate [T, n] with any row stride, one dtype."""
    _need_cuda(y, gate)
    if y.dim() != 2 or tuple(gate.shape) != tuple(y.shape) or gate.dtype != y.dtype or gate.stride(1) != 1:
        raise KernelError("sigmoid_gate: y [T, n], gate [T, n] of the same dtype with contiguous rows")
    _contig("y", y)
    f = _fn("latent", "il_sigmoid_gate", [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(y), kind_of(y.dtype), _ptr(gate), gate.stride(0), y.shape[0], y.shape[1], _stream()), "sigmoid_gate")


MOE_MAX_TOP = 32
ROUTE_TOP_LOGITS, ROUTE_SOFTMAX_ALL = 0, 1         # how a router's logits become choices and weights (`moe_select`)


def moe_route(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], idx: torch.Tensor, wt: torch.Tensor, top: int,
              norm_in: Optional["NormedInput"] = None, rstd_out: Optional[torch.Tensor] = None) -> None:
    """Per row of x [T,H]: logits = x w^T + bias in f32, the `top` largest experts into idx [T, top] (int32), the softmax
    over the chosen logits into wt [T, top] (float32).
    norm_in: x is `norm_in.xw`, rows whose RMSNorm is not finished; the router multiplies them by rstd itself (in f32) and
    leaves rstd [T] in `rstd_out` (float32) for the products that read the same rows."""
    _need_cuda(x, w, bias, idx, wt, rstd_out)
    T, H = x.shape
    E = w.shape[0]
    if w.dtype != x.dtype or w.shape[1] != H or x.stride(1) != 1 or not w.is_contiguous():
        raise KernelError("moe_route: x [T,H], w [E,H] of the same dtype")
    if idx.dtype != torch.int32 or wt.dtype != torch.float32 or tuple(idx.shape) != (T, top) or tuple(wt.shape) != (T, top):
        raise KernelError("moe_route: idx int32 [T, top], wt float32 [T, top]")
    if not 0 < top <= min(E, MOE_MAX_TOP):
        raise KernelError(f"moe_route: top must be in 1..min(experts, {MOE_MAX_TOP})")
    if bias is not None and bias.numel() != E:
        raise KernelError("moe_route: bias [E]")
    _contig("idx", idx), _contig("wt", wt)
    if rstd_out is not None and (rstd_out.dtype != torch.float32 or rstd_out.numel() < T or not rstd_out.is_contiguous()):
        raise KernelError("moe_route: rstd_out float32 [T]")
    if norm_in is not None and norm_in.width != H:
        raise KernelError("moe_route: norm_in is of another width")
    sq, n_partial, _, eps = _norm_args(norm_in, T)
    f = _fn("moe", "il_moe_route", [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                                    _c_int, _c_void_p, _c_int, _c_float, _c_void_p, _c_void_p])
    _check(f(_ptr(x), kind_of(x.dtype), x.stride(0), _ptr(w), _ptr(bias), kind_of(bias.dtype) if bias is not None else 0, _ptr(idx),
             _ptr(wt), T, H, E, top, sq, n_partial, eps, _ptr(rstd_out), _stream()), "moe_route")


def moe_route_sort_small(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], z: torch.Tensor, idx: torch.Tensor, wt: torch.Tensor,
                         top: int, group_off: torch.Tensor, pos_of_slot: torch.Tensor, row_of_pos: torch.Tensor,
                         norm_in: Optional["NormedInput"] = None, rstd_out: Optional[torch.Tensor] = None, extra: int = 0,
                         rule: int = ROUTE_TOP_LOGITS, out_scale: float = 1.0) -> None:
    """`moe_route` and `moe_sort` for a few bfloat16 rows (a decode step) as two short kernels: the logits, a warp per
    (token, expert), into z [T, E + extra] float32; then one block that chooses for every token and sorts the slots.
    Rows of whole 16-byte chunks (H a multiple of 8); `route_sort_small_ok` says whether a shape is taken.
    `extra`: the last rows of `w` are no experts - their products are written to z's last columns and take no part in the
    choice. `rule`, `out_scale`: see `moe_select`."""
    _need_cuda(x, w, bias, z, idx, wt, group_off, pos_of_slot, row_of_pos, rstd_out)
    T, H = x.shape
    E = w.shape[0] - extra
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != H or x.stride(1) != 1 or not w.is_contiguous():
        raise KernelError("moe_route_sort_small: bfloat16 x [T,H], w [E,H]")
    if z.dtype != torch.float32 or z.numel() < T * (E + extra) or not z.is_contiguous():
        raise KernelError("moe_route_sort_small: z float32 [T, E + extra]")
    if idx.dtype != torch.int32 or wt.dtype != torch.float32 or tuple(idx.shape) != (T, top) or tuple(wt.shape) != (T, top):
        raise KernelError("moe_route_sort_small: idx int32 [T, top], wt float32 [T, top]")
    if not 0 < top <= min(E, MOE_MAX_TOP) or (bias is not None and bias.numel() != E):
        raise KernelError(f"moe_route_sort_small: top in 1..min(experts, {MOE_MAX_TOP}), bias [E]")
    for t in (group_off, pos_of_slot, row_of_pos):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("moe_route_sort_small: contiguous int32 tensors")
    if group_off.numel() < E + 1 or pos_of_slot.numel() < T * top or row_of_pos.numel() < T * top:
        raise KernelError("moe_route_sort_small: group_off [E + 1], pos_of_slot and row_of_pos [T * top]")
    if rstd_out is not None and (rstd_out.dtype != torch.float32 or rstd_out.numel() < T or not rstd_out.is_contiguous()):
        raise KernelError("moe_route_sort_small: rstd_out float32 [T]")
    if norm_in is not None and norm_in.width != H:
        raise KernelError("moe_route_sort_small: norm_in is of another width")
    _contig("idx", idx), _contig("wt", wt)
    sq, n_partial, _, eps = _norm_args(norm_in, T)
    f = _fn("moe", "il_moe_route_sort_small", [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                                               _c_int, _c_int, _c_void_p, _c_int, _c_float, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                               _c_int, _c_float, _c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), _ptr(bias), kind_of(bias.dtype) if bias is not None else 0, _ptr(z), _ptr(idx), _ptr(wt), T, H, E,
             top, sq, n_partial, eps, _ptr(rstd_out), _ptr(group_off), _ptr(pos_of_slot), _ptr(row_of_pos), int(extra), int(rule),
             float(out_scale), _stream()), "moe_route_sort_small")
    count_launches(1)                             # two kernels


def route_sort_small_ok(T: int, H: int, E: int) -> bool:
    """Up to 16 rows: beyond, the one block that chooses for every token takes longer than a block a token does
    (measured at 64 rows, 64 experts: 5.2 + 14.7 us against 11.2 + 3.5 us)."""
    return 0 < T <= SKINNY_MAX_ROWS and H % 8 == 0 and 34 * E * 4 <= 200 * 1024


def moe_select(z: torch.Tensor, bias: Optional[torch.Tensor], idx: torch.Tensor, wt: torch.Tensor, top: int,
               rule: int = ROUTE_TOP_LOGITS, out_scale: float = 1.0) -> None:
    """The choice of `moe_route` for logits a matrix product has written: z [T, E] float32 (+ bias [E]) -> idx, wt [T, top].
    rule ROUTE_TOP_LOGITS: the `top` largest of z + bias, their weights the softmax over the chosen alone.
    rule ROUTE_SOFTMAX_ALL: scores s = softmax(z) over all E; the `top` largest of s + bias are chosen (the lower expert wins a
    tie); the weights are the chosen experts' s over their sum (+ 1e-20), times out_scale."""
    _need_cuda(z, bias, idx, wt)
    T, E = z.shape
    if z.dtype != torch.float32 or z.stride(1) != 1:
        raise KernelError("moe_select: z float32 [T, E] with contiguous rows")
    if idx.dtype != torch.int32 or wt.dtype != torch.float32 or tuple(idx.shape) != (T, top) or tuple(wt.shape) != (T, top):
        raise KernelError("moe_select: idx int32 [T, top], wt float32 [T, top]")
    if not 0 < top <= min(E, MOE_MAX_TOP):
        raise KernelError(f"moe_select: top must be in 1..min(experts, {MOE_MAX_TOP})")
    if bias is not None and bias.numel() != E:
        raise KernelError("moe_select: bias [E]")
    _contig("idx", idx), _contig("wt", wt)
    f = _fn("moe", "il_moe_select", [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float,
                                     _c_void_p])
    _check(f(_ptr(z), z.stride(0), _ptr(bias), kind_of(bias.dtype) if bias is not None else 0, _ptr(idx), _ptr(wt), T, E, top, int(rule),
             float(out_scale), _stream()), "moe_select")


def moe_sort(idx: torch.Tensor, n_experts: int, group_off: torch.Tensor, pos_of_slot: torch.Tensor, row_of_pos: torch.Tensor) -> None:
    """Orders the slots (token, choice) of idx [T, top] by expert: group_off [E + 1], pos_of_slot [T * top], row_of_pos [T * top]."""
    _need_cuda(idx, group_off, pos_of_slot, row_of_pos)
    T, top = idx.shape
    for t in (idx, group_off, pos_of_slot, row_of_pos):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("moe_sort: contiguous int32 tensors")
    if group_off.numel() < n_experts + 1 or pos_of_slot.numel() < T * top or row_of_pos.numel() < T * top:
        raise KernelError("moe_sort: outputs too small")
    f = _fn("moe", "il_moe_sort", [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p])
    _check(f(_ptr(idx), T * top, top, n_experts, _ptr(group_off), _ptr(pos_of_slot), _ptr(row_of_pos), _stream()), "moe_sort")


def gather_rows(x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """out[p] = x[rows[p]] for the len(out) first entries of rows (int32 on the device)."""
    _need_cuda(x, rows, out)
    n, H = out.shape
    if x.dtype != out.dtype or x.shape[1] != H or x.stride(1) != 1 or rows.dtype != torch.int32 or rows.numel() < n:
        raise KernelError("gather_rows: x [*, H], out [n, H] of one dtype, rows int32 [n]")
    _contig("out", out)
    f = _fn("moe", "il_gather_rows", [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(x), kind_of(x.dtype), x.stride(0), _ptr(rows), _ptr(out), n, H, _stream()), "gather_rows")


def moe_combine(y: torch.Tensor, pos_of_slot: torch.Tensor, wt: torch.Tensor, shared_rows: Optional[torch.Tensor], out: torch.Tensor, *,
                group_off: Optional[torch.Tensor] = None, n_real: int = 0, x: Optional[torch.Tensor] = None,
                shared_gate: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum_k wt[t,k] * y[pos_of_slot[t*top + k]] (+ shared_rows[t]), summed in f32 in the order of k.
    With `group_off` (int32, the sorted order's group starts), `n_real` and `x` [T, H]: the experts from n_real on have no
    weights and return their input - a choice whose place is group_off[n_real] or later adds wt * x[t] instead of a row of y.
    `shared_gate`: float32 [T] (any stride) - the shared row is multiplied by its sigmoid."""
    _need_cuda(y, pos_of_slot, wt, shared_rows, out, group_off, x, shared_gate)
    T, top = wt.shape
    H = out.shape[1]
    if group_off is not None and (x is None or x.dtype != out.dtype or tuple(x.shape) != (T, H) or x.stride(1) != 1
                                  or group_off.dtype != torch.int32 or group_off.numel() <= n_real):
        raise KernelError("moe_combine: identity experts need group_off int32 [> n_real] and x [T, H] of out's dtype")
    if shared_gate is not None and (shared_gate.dtype != torch.float32 or shared_gate.dim() != 1 or shared_gate.numel() != T):
        raise KernelError("moe_combine: shared_gate float32 [T]")
    if y.dtype != out.dtype or y.shape[1] != H or out.shape[0] != T or y.shape[0] < T * top:
        raise KernelError("moe_combine: y [T * top, H], out [T, H] of the same dtype")
    if shared_rows is not None and (shared_rows.dtype != out.dtype or tuple(shared_rows.shape) != (T, H)):
        raise KernelError("moe_combine: shared_rows [T, H]")
    _contig("y", y), _contig("out", out), _contig("wt", wt)
    if shared_rows is not None:
        _contig("shared_rows", shared_rows)
    f = _fn("moe", "il_moe_combine", [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int,
                                      _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p])
    _check(f(_ptr(y), kind_of(y.dtype), _ptr(pos_of_slot), _ptr(wt), _ptr(shared_rows), _ptr(out), T, H, top, _ptr(group_off), int(n_real),
             _ptr(x), 0 if x is None else x.stride(0), _ptr(shared_gate), 0 if shared_gate is None else shared_gate.stride(0), _stream()),
           "moe_combine")


def moe_combine_resid(y: torch.Tensor, pos_of_slot: torch.Tensor, wt: torch.Tensor, shared_rows: Optional[torch.Tensor], resid: torch.Tensor,
                      branch_scale: float, norm_weight: torch.Tensor, eps: float, xw: torch.Tensor, sumsq: torch.Tensor) -> NormedInput:
    """`moe_combine` as the last step of a branch of a few bfloat16 rows, with the residual add and the next RMSNorm's
    inputs: resid (float32 [T,H], in place) += branch_scale * bf16(sum); xw = resid * norm_weight; sumsq[t][b] = sum of
    resid[t]^2 over columns 16b..16b+15. Returns what the next product needs to finish the norm."""
    _need_cuda(y, pos_of_slot, wt, shared_rows, resid, norm_weight, xw, sumsq)
    T, top = wt.shape
    H = resid.shape[1]
    nb = (H + 15) // 16
    if y.dtype != torch.bfloat16 or y.shape[1] != H or y.shape[0] < T * top or H % 4:
        raise KernelError("moe_combine_resid: y bfloat16 [T * top, H], H a multiple of 4")
    if shared_rows is not None and (shared_rows.dtype != torch.bfloat16 or tuple(shared_rows.shape) != (T, H)):
        raise KernelError("moe_combine_resid: shared_rows bfloat16 [T, H]")
    if resid.dtype != torch.float32 or tuple(resid.shape) != (T, H) or xw.dtype != torch.bfloat16 or tuple(xw.shape) != (T, H):
        raise KernelError("moe_combine_resid: resid float32 [T,H], xw bfloat16 [T,H]")
    if sumsq.dtype != torch.float32 or tuple(sumsq.shape) != (T, nb) or nb > NORM_MAX_BLOCKS or norm_weight.numel() != H:
        raise KernelError("moe_combine_resid: sumsq float32 [T, ceil(H/16) <= 256], norm_weight [H]")
    _contig("y", y), _contig("wt", wt), _contig("resid", resid), _contig("xw", xw), _contig("sumsq", sumsq), _contig("norm_weight", norm_weight)
    if shared_rows is not None:
        _contig("shared_rows", shared_rows)
    f = _fn("moe", "il_moe_combine_resid", [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_float, _c_void_p,
                                            _c_int, _c_void_p, _c_void_p, _c_void_p])
    _check(f(_ptr(y), _ptr(pos_of_slot), _ptr(wt), _ptr(shared_rows), T, H, top, _ptr(resid), branch_scale, _ptr(norm_weight),
             kind_of(norm_weight.dtype), _ptr(xw), _ptr(sumsq), _stream()), "moe_combine_resid")
    return NormedInput(xw, sumsq, H, eps)


def gemm_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, group_off: Optional[torch.Tensor] = None,
                 a_rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None, glu: bool = False,
                 gate: Optional[torch.Tensor] = None, row_scale: Optional[torch.Tensor] = None) -> None:
    """Products over groups, out_g = a_g w_g^T, w [G, N, K] (glu: [G, 2N, K], gate rows then up rows, out = silu(gate) * up).
    Ragged (`group_off` int32 [G + 1] on the device): the `n_rows` rows of `out` [n_rows, N] stand sorted by group, group g
    owning places group_off[g] .. group_off[g+1] - 1; the row of `a` [*, K] at a place is a_rows[place] (or the place).
    Batched (no `group_off`): a [M, G, K] and out [M, G, N] are column ranges of shared rows; `gate` [M, G, N] multiplies
    out by its sigmoid.
    row_scale (ragged, bfloat16 rows of 16-byte chunks): float32 per row of `a`; the products of a row are multiplied by
    its factor before the epilogue (the rstd of a norm the rows have not been divided by)."""
    _need_cuda(a, w, out, group_off, a_rows, gate, row_scale)
    if row_scale is not None and (group_off is None or row_scale.dtype != torch.float32 or not row_scale.is_contiguous()
                                  or row_scale.numel() < a.shape[0]):
        raise KernelError("gemm_grouped: row_scale float32 [rows of a], with the ragged form")
    if w.dim() != 3 or not w.is_contiguous() or w.dtype != a.dtype or out.dtype != a.dtype:
        raise KernelError("gemm_grouped: w [G, N, K] contiguous, one dtype for a, w and out")
    G, K = w.shape[0], w.shape[2]
    N = w.shape[1] // 2 if glu else w.shape[1]
    if group_off is not None:
        M = int(n_rows if n_rows is not None else out.shape[0])
        if a.dim() != 2 or a.shape[1] != K or a.stride(1) != 1 or out.dim() != 2 or out.shape[1] != N or out.shape[0] < M or out.stride(1) != 1:
            raise KernelError(f"gemm_grouped: ragged a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
        if group_off.dtype != torch.int32 or group_off.numel() < G + 1 or (a_rows is not None and (a_rows.dtype != torch.int32 or a_rows.numel() < M)):
            raise KernelError("gemm_grouped: group_off int32 [G + 1], a_rows int32 [rows]")
        if a_rows is None and a.shape[0] < M:
            raise KernelError("gemm_grouped: a has fewer rows than places")
        if gate is not None:
            raise KernelError("gemm_grouped: gate goes with the batched form")
        lda, a_gs, ldc, c_gs, ldg, g_gs = a.stride(0), 0, out.stride(0), 0, 0, 0
    else:
        if a.dim() != 3 or out.dim() != 3 or a.shape[1] != G or out.shape[1] != G or a.shape[2] != K or out.shape[2] != N or a.shape[0] != out.shape[0]:
            raise KernelError(f"gemm_grouped: batched a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
        if a.stride(2) != 1 or out.stride(2) != 1:
            raise KernelError("gemm_grouped: innermost dimension must be contiguous")
        M = a.shape[0]
        lda, a_gs, ldc, c_gs = a.stride(0), a.stride(1), out.stride(0), out.stride(1)
        ldg = g_gs = 0
        if gate is not None:
            if tuple(gate.shape) != tuple(out.shape) or gate.dtype != out.dtype or gate.stride(2) != 1:
                raise KernelError("gemm_grouped: gate [M, G, N] of out's dtype")
            ldg, g_gs = gate.stride(0), gate.stride(1)
    f = _fn("gemm_grouped", "il_gemm_grouped", [_c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_void_p, _c_int, _c_ll, _c_void_p, _c_int,
                                                _c_ll, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_ll,
                                                _c_void_p, _c_void_p])
    _check(f(_ptr(a), kind_of(a.dtype), lda, a_gs, _ptr(a_rows), _ptr(w), w.stride(1), w.stride(0), _ptr(out), ldc, c_gs, _ptr(group_off),
             G, M, N, K, int(glu), _ptr(gate), ldg, g_gs, _ptr(row_scale), _stream()), "gemm_grouped")


# ----------------------------------------------------------------------------------------------
def _np_ptr(a) -> _c_void_p:
    return _c_void_p(a.ctypes.data)


def step_fill(out, out_cap: int, E: int, Ep: int, Tp: int, order, n_tok, start, slot, fresh, tokens, tok_off, widths, tbl_ptr,
              tbl_len, scratch_page, scratch_slot: int, want, want_off, pad_at: int, n_want_fixed: int, n_patch_cap: int, offsets,
              outs) -> int:
    """Native host code (csrc/step_fill.cpp): fills a step's descriptors into the int32 host array `out` from columns
    given as numpy arrays (int32 unless said: `fresh` uint8, `tokens` int64, `tbl_ptr` uint64 addresses of the block
    tables' arrays). The Ep - E padding entries of a step that is replayed as a graph run behind the first `pad_at`
    entries; `n_want_fixed` is such a step's number of wanted rows (-1: as many as are asked for). `offsets` (int32 [12]) receives where each part starts, `outs` (int32 [3]) the number of device
    tokens, of wanted rows, and the entry at fault. Returns 0 or the negative code of the fault."""
    for name, a, dt in (("order", order, "int32"), ("n_tok", n_tok, "int32"), ("start", start, "int32"), ("slot", slot, "int32"),
                        ("fresh", fresh, "uint8"), ("tokens", tokens, "int64"), ("tok_off", tok_off, "int32"),
                        ("widths", widths, "int32"), ("tbl_ptr", tbl_ptr, "uint64"), ("tbl_len", tbl_len, "int32"),
                        ("scratch_page", scratch_page, "int32"), ("want", want, "int32"), ("want_off", want_off, "int32"),
                        ("offsets", offsets, "int32"), ("outs", outs, "int32"), ("out", out, "int32")):
        if a.dtype.name != dt or not a.flags["C_CONTIGUOUS"]:
            raise KernelError(f"step_fill: {name} must be a contiguous {dt} array")
    if (len(order) != E or len(n_tok) != E or len(start) != E or len(slot) != E or len(fresh) != E or len(tok_off) != E + 1
            or len(want_off) != E + 1 or tbl_ptr.size != widths.size * E or tbl_len.size != widths.size * E
            or scratch_page.size != widths.size or offsets.size < 12 or outs.size < 3 or out.size < out_cap):
        raise KernelError("step_fill: array sizes do not match the number of entries and groups")
    lib = build.load("step_fill")
    f = lib.il_step_fill
    if not getattr(f, "_sig", False):
        f.argtypes = ([_c_void_p, ctypes.c_longlong, _c_int, _c_int, _c_int] + [_c_void_p] * 7 + [_c_int] + [_c_void_p] * 4 + [_c_int]
                      + [_c_void_p] * 2 + [_c_int, _c_int, _c_int] + [_c_void_p] * 4)
        f.restype = _c_int
        f._sig = True
    return int(f(_np_ptr(out), out_cap, E, Ep, Tp, _np_ptr(order), _np_ptr(n_tok), _np_ptr(start), _np_ptr(slot), _np_ptr(fresh),
                 _np_ptr(tokens), _np_ptr(tok_off), int(widths.size), _np_ptr(widths), _np_ptr(tbl_ptr), _np_ptr(tbl_len),
                 _np_ptr(scratch_page), scratch_slot, _np_ptr(want), _np_ptr(want_off), int(pad_at), int(n_want_fixed), n_patch_cap,
                 _c_void_p(offsets.ctypes.data), _c_void_p(outs.ctypes.data), _c_void_p(outs.ctypes.data + 4),
                 _c_void_p(outs.ctypes.data + 8)))


# ---- sequence mixers with a state of fixed size (csrc/seqmix.cu) ---------------------------------------------------------
def _i32(name: str, *ts: torch.Tensor) -> None:
    for t in ts:
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError(f"{name}: descriptors must be contiguous int32 tensors")


def short_conv(x: torch.Tensor, x_off: int, w: torch.Tensor, state: torch.Tensor, st_off: int, read_slots: torch.Tensor,
               tok_entry: torch.Tensor, entry_qstart: torch.Tensor, out: torch.Tensor, out_off: int, n_seg: int, seg_in: int,
               seg_out: int, act: int = 0, n_seg2: int = 0, seg_in2: int = 0, write_slots: Optional[torch.Tensor] = None) -> None:
    """Causal convolution over time of n_seg * seg_in (+ n_seg2 * seg_in2) channels of `x` (columns from x_off), per channel,
    with weights w float32 [channels, taps] whose last column meets the current token. Inputs before a step's first row come
    from `state` (float32 [slots, taps-1, all channels], this call's channels from column st_off; slot read_slots[entry]).
    Written to `out` from column out_off as segments of seg_out columns each, the surplus zero. act 1: silu.
    `write_slots`: entries that bring ONE token have their state moved on here, in slot write_slots[entry] (the thread that
    reads such an entry's state is the only one that does); `short_conv_state` then only has the other entries to do."""
    _need_cuda(x, w, state, read_slots, tok_entry, entry_qstart, out, write_slots)
    _i32("short_conv", read_slots, tok_entry, entry_qstart)
    if write_slots is not None:
        _i32("short_conv", write_slots)
    T, taps = x.shape[0], w.shape[1]
    n_ch = n_seg * seg_in + n_seg2 * seg_in2
    if w.dtype != torch.float32 or not w.is_contiguous() or w.shape[0] != n_ch:
        raise KernelError("short_conv: w float32 [channels, taps]")
    if state.dtype != torch.float32 or not state.is_contiguous() or state.dim() != 3 or state.shape[1] != max(taps - 1, 1):
        raise KernelError("short_conv: state float32 [slots, taps-1, channels]")
    if (x.stride(1) != 1 or out.stride(1) != 1 or out.shape[0] != T or x_off + n_ch > x.shape[1]
            or out_off + (n_seg + n_seg2) * seg_out > out.shape[1] or st_off + n_ch > state.shape[2]):
        raise KernelError("short_conv: column ranges do not fit")
    f = _fn("seqmix", "il_short_conv", [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_ll, _c_int, _c_int,
                                        _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                                        _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(x), kind_of(x.dtype), x.stride(0), x_off, _ptr(w), taps, _ptr(state), state.stride(0), st_off, state.shape[2],
             _ptr(read_slots), _ptr(write_slots if taps > 1 else None), _ptr(tok_entry), _ptr(entry_qstart), _ptr(out), kind_of(out.dtype),
             out.stride(0), out_off, n_seg, seg_in, n_seg2, seg_in2, seg_out, act, T, _stream()), "short_conv")


def short_conv_state(x: torch.Tensor, x_off: int, n_channels: int, taps: int, state: torch.Tensor, st_off: int,
                     read_slots: torch.Tensor, write_slots: torch.Tensor, entry_qstart: torch.Tensor, n_entries: int,
                     first_entry: int = 0) -> None:
    """The convolution's state after the step: the last taps-1 inputs of entries first_entry .. first_entry + n_entries - 1,
    into slot write_slots[entry]."""
    if taps <= 1 or n_entries <= 0:
        return
    _need_cuda(x, state, read_slots, write_slots, entry_qstart)
    _i32("short_conv_state", read_slots, write_slots, entry_qstart)
    if state.dtype != torch.float32 or not state.is_contiguous() or state.dim() != 3 or state.shape[1] != taps - 1:
        raise KernelError("short_conv_state: state float32 [slots, taps-1, channels]")
    if x.stride(1) != 1 or x_off + n_channels > x.shape[1] or st_off + n_channels > state.shape[2]:
        raise KernelError("short_conv_state: column ranges do not fit")
    f = _fn("seqmix", "il_short_conv_state", [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_ll, _c_int, _c_int,
                                              _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(x), kind_of(x.dtype), x.stride(0), x_off, n_channels, taps, _ptr(state), state.stride(0), st_off, state.shape[2],
             _ptr(read_slots), _ptr(write_slots), _ptr(entry_qstart), n_entries, first_entry, _stream()), "short_conv_state")


def delta_prep(qk: torch.Tensor, q_off: int, k_off: int, n_qk_heads: int, dim: int, q_scale: float, unit_eps: float,
               ab: torch.Tensor, b_off: int, a_off: int, a_log: torch.Tensor, dt_bias: torch.Tensor, beta: torch.Tensor,
               gdec: torch.Tensor, n_heads: int) -> None:
    """In place: the q and k heads of `qk` (float32) become unit vectors, x / sqrt(sum x^2 + unit_eps), q also times q_scale.
    beta[t,h] = sigmoid(ab[t, b_off+h]); gdec[t,h] = exp(-exp(a_log[h]) * softplus(ab[t, a_off+h] + dt_bias[h]))."""
    _need_cuda(qk, ab, a_log, dt_bias, beta, gdec)
    T = qk.shape[0]
    for t in (qk, ab, a_log, dt_bias, beta, gdec):
        if t.dtype != torch.float32:
            raise KernelError("delta_prep: float32 tensors")
    if (qk.stride(1) != 1 or ab.stride(1) != 1 or a_log.numel() != n_heads or dt_bias.numel() != n_heads
            or tuple(beta.shape) != (T, n_heads) or tuple(gdec.shape) != (T, n_heads) or not beta.is_contiguous() or not gdec.is_contiguous()):
        raise KernelError("delta_prep: shapes")
    f = _fn("seqmix", "il_delta_prep", [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_void_p, _c_int, _c_int,
                                        _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(qk), qk.stride(0), q_off, k_off, n_qk_heads, dim, q_scale, unit_eps, _ptr(ab), ab.stride(0), b_off, a_off,
             _ptr(a_log), _ptr(dt_bias), _ptr(beta), _ptr(gdec), n_heads, T, _stream()), "delta_prep")


SCAN_DECAY, SCAN_DELTA, SCAN_GATED, SCAN_CHANNEL_DECAY = 0, 1, 3, 4


def matrix_state_scan(mode: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, n_heads: int, n_qk_heads: int, dim: int,
                      vdim: int, in_act: int, decay: Optional[torch.Tensor], beta: Optional[torch.Tensor],
                      gdec: Optional[torch.Tensor], state: torch.Tensor, read_slots: torch.Tensor, write_slots: torch.Tensor,
                      entry_qstart: torch.Tensor, n_entries: int, out: torch.Tensor, generic: bool = False, first_entry: int = 0,
                      single: bool = False, seg_len: int = 0, n_tiles: int = 0, seg_state: Optional[torch.Tensor] = None) -> None:
    """A recurrence over a float32 state S [dim, vdim] per (request, head), token by token in each entry's order.
    SCAN_DECAY: S = decay[h] S + k v^T, o = S^T q. SCAN_DELTA: S = g S; u = beta (v - S^T k); S += k u^T; o = S^T q.
    SCAN_GATED: S = g S + beta k [v, 1]^T, o = S^T q with g, beta per token and head (`gdec`, `beta`); the state and the output
    have one column more than v (`vdim` counts it: v heads are vdim - 1 wide), fed by the constant 1.
    SCAN_CHANNEL_DECAY: o = (S + diag(u_h) k v^T)^T q, then S = diag(w_t) S + k v^T: `gdec` holds w, float32 [T, >= heads*dim]
    (a decay per token, head and key channel; a view with a row stride), `decay` the bonus u, float32 [heads, dim].
    q, k float32 [T, >= n_qk_heads*dim] (views with a row stride), v float32 [T, >= n_heads*vdim], out float32 [T, n_heads*vdim];
    value head h reads q/k head h // (n_heads // n_qk_heads). in_act 1: silu on q, k, v as read.
    state float32 [slots, n_heads, vdim, dim] (S column by column: the dim entries behind one output lie together). `generic`: the kernel that keeps the state in shared memory (any size; the
    one that runs beyond a key size of 256) instead of the one that keeps it in registers. Entries first_entry ..
    first_entry + n_entries - 1 are run; `single`: each of them brings one token (the form made for decoding).
    seg_len > 0 (SCAN_DECAY, key sizes up to 256): every entry's tokens are walked in segments of seg_len at once, each from
    nothing, and a second launch adds what the state at a segment's start contributes (the sum is linear in it);
    `n_tiles` bounds the number of segments, `seg_state` is float32 scratch of n_tiles * heads * vdim * dim."""
    _need_cuda(q, k, v, decay, beta, gdec, state, read_slots, write_slots, entry_qstart, out)
    _i32("matrix_state_scan", read_slots, write_slots, entry_qstart)
    for t in (q, k, v, out, state):
        if t.dtype != torch.float32 or t.stride(-1) != 1:
            raise KernelError("matrix_state_scan: float32 tensors with contiguous rows")
    if not state.is_contiguous() or tuple(state.shape[1:]) != (n_heads, vdim, dim):
        raise KernelError("matrix_state_scan: state float32 [slots, heads, vdim, dim]")
    v_cols = n_heads * (vdim - 1 if mode == SCAN_GATED else vdim)
    if out.shape[1] != n_heads * vdim or q.shape[1] < n_qk_heads * dim or k.shape[1] < n_qk_heads * dim or v.shape[1] < v_cols:
        raise KernelError("matrix_state_scan: shapes")
    ld_g = 0
    if mode == SCAN_CHANNEL_DECAY:
        if (gdec is None or decay is None or gdec.dtype != torch.float32 or gdec.stride(-1) != 1 or gdec.shape[1] < n_heads * dim
                or decay.dtype != torch.float32 or not decay.is_contiguous() or decay.numel() != n_heads * dim or n_qk_heads != n_heads):
            raise KernelError("matrix_state_scan: channel decays float32 [T, heads*dim], bonus float32 [heads, dim], as many q/k heads as heads")
        ld_g = gdec.stride(0)
    if seg_len > 0:
        _need_cuda(seg_state)
        if (mode != SCAN_DECAY or generic or single or dim > 256 or seg_len % 8 or n_tiles <= 0 or seg_state is None
                or seg_state.dtype != torch.float32 or not seg_state.is_contiguous() or seg_state.numel() < n_tiles * n_heads * vdim * dim):
            raise KernelError("matrix_state_scan: segments go with SCAN_DECAY in the register form and float32 scratch for n_tiles states")
    f = _fn("seqmix", "il_matrix_state_scan", [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                               _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_ll, _c_void_p, _c_void_p,
                                               _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                               _c_void_p])
    _check(f(mode, _ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), v.stride(0), n_heads, n_qk_heads, dim, vdim, in_act,
             _ptr(decay), _ptr(beta), _ptr(gdec), _ptr(state), state.stride(0), _ptr(read_slots), _ptr(write_slots),
             _ptr(entry_qstart), n_entries, _ptr(out), out.stride(0), int(generic), first_entry, int(single), seg_len, n_tiles,
             _ptr(seg_state), ld_g, _stream()), "matrix_state_scan")
    if seg_len > 0:
        count_launches(1)                         # the second pass


def matrix_state_scan_step(ctx, *args, **kw) -> None:
    """`matrix_state_scan` over a step's entries: the single tokens (the first `ctx.n_decode` entries) by the form made for
    them, the prompt portions behind them by the chunked form - the decayed sum of long portions in segments that run at
    once (`SCAN_SEGMENT` tokens; the choice rests on the step's shape alone, so a replayed step makes it the same way)."""
    n_dec, E = ctx.n_decode, ctx.n_entries
    if n_dec > 0:
        matrix_state_scan(*args, n_entries=n_dec, first_entry=0, single=True, **kw)
    if E > n_dec:
        mode, dim, vdim, n_heads = args[0], args[6], args[7], args[4]
        if (mode == SCAN_DECAY and not kw.get("generic") and dim <= 256 and ctx.T - n_dec >= 2 * SCAN_SEGMENT):
            n_tiles = ctx.prompt_tiles(SCAN_SEGMENT)
            scratch = ctx.ws.flat("scan_segment_state", n_tiles * n_heads * vdim * dim, torch.float32)
            matrix_state_scan(*args, n_entries=E - n_dec, first_entry=n_dec, single=False, seg_len=SCAN_SEGMENT, n_tiles=n_tiles,
                              seg_state=scratch, **kw)
        else:
            matrix_state_scan(*args, n_entries=E - n_dec, first_entry=n_dec, single=False, **kw)


SCAN_SEGMENT = 128


def token_shift_mix(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, read_slots: torch.Tensor, write_slots: Optional[torch.Tensor],
                    tok_entry: torch.Tensor, entry_qstart: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, m*W + c] = h[t, c] + (h_prev[t, c] - h[t, c]) * mu[m, c]: the blends of a token's row with the row before it in its
    sequence, one per row of `mu` (float32 [n_mix, W]). The row before a step's first token is the request's state (float32
    [slots, W]; the zero slot for a sequence's first token), which receives the entry's last row (`write_slots` None: not)."""
    _need_cuda(h, mu, state, read_slots, write_slots, tok_entry, entry_qstart, out)
    _i32("token_shift_mix", read_slots, tok_entry, entry_qstart)
    T, W = h.shape
    n_mix = mu.shape[0]
    if mu.dtype != torch.float32 or not mu.is_contiguous() or mu.shape[1] != W or h.stride(1) != 1:
        raise KernelError("token_shift_mix: mu float32 [n_mix, W], h [T, W] with contiguous rows")
    if out.dtype != h.dtype or tuple(out.shape) != (T, n_mix * W) or out.stride(1) != 1:
        raise KernelError("token_shift_mix: out [T, n_mix * W] of h's dtype")
    if state.dtype != torch.float32 or not state.is_contiguous() or state.dim() != 2 or state.shape[1] != W:
        raise KernelError("token_shift_mix: state float32 [slots, W]")
    f = _fn("seqmix", "il_token_shift_mix", [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_void_p,
                                             _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(h), kind_of(h.dtype), h.stride(0), _ptr(mu), n_mix, _ptr(state), state.stride(0), _ptr(read_slots), _ptr(write_slots),
             _ptr(tok_entry), _ptr(entry_qstart), _ptr(out), out.stride(0), W, T, _stream()), "token_shift_mix")


def double_exp_decay(z: torch.Tensor, w0: Optional[torch.Tensor], cols: int) -> None:
    """z[:, :cols] = exp(-exp(z[:, :cols] + w0)) in place: float32 rows, w0 float32 [cols] or None."""
    _need_cuda(z, w0)
    if z.dtype != torch.float32 or z.dim() != 2 or z.stride(1) != 1 or cols > z.shape[1]:
        raise KernelError("double_exp_decay: float32 [T, >= cols] with contiguous rows")
    if w0 is not None and (w0.dtype != torch.float32 or w0.numel() != cols or not w0.is_contiguous()):
        raise KernelError("double_exp_decay: w0 float32 [cols]")
    f = _fn("seqmix", "il_double_exp_decay", [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(z), z.stride(0), _ptr(w0), cols, z.shape[0], _stream()), "double_exp_decay")


def tanh_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = tanh(x): x contiguous float32, out contiguous float32 or bfloat16 of the same shape."""
    _need_cuda(x, out)
    if x.dtype != torch.float32 or x.shape != out.shape:
        raise KernelError("tanh_rows: float32 in, one shape")
    _contig("x", x), _contig("out", out)
    f = _fn("seqmix", "il_tanh_rows", [_c_void_p, _c_void_p, _c_int, _c_ll, _c_void_p])
    _check(f(_ptr(x), _ptr(out), kind_of(out.dtype), x.numel(), _stream()), "tanh_rows")


def silu_cols(x: torch.Tensor, cols: int) -> None:
    """x[:, :cols] = silu(x[:, :cols]) in place, float32 rows (the same SiLU the recurrence kernels apply to their inputs)."""
    _need_cuda(x)
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1 or cols > x.shape[1]:
        raise KernelError("silu_cols: float32 [T, >= cols] with contiguous rows")
    f = _fn("seqmix", "il_silu_cols", [_c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(x), x.stride(0), cols, x.shape[0], _stream()), "silu_cols")


def stabilized_gates(z: torch.Tensor, i_off: int, f_off: int, cap: float, m_state: torch.Tensor, read_slots: torch.Tensor,
                     write_slots: torch.Tensor, entry_qstart: torch.Tensor, n_entries: int, decay: torch.Tensor, in_weight: torch.Tensor,
                     den_floor: torch.Tensor, n_heads: int, first_entry: int = 0) -> None:
    """Log-space gates of a matrix memory with their running maximum m (part of the request's state, float32 [slots, heads]):
    i = cap tanh(z[:, i_off + h] / cap), f = logsigmoid(cap tanh(z[:, f_off + h] / cap)) (cap <= 0: no cap);
    m_t = max(f_t + m_(t-1), i_t); decay = exp(f + m_(t-1) - m_t), in_weight = exp(i - m_t), den_floor = exp(-m_t): float32 [T, heads]."""
    _need_cuda(z, m_state, read_slots, write_slots, entry_qstart, decay, in_weight, den_floor)
    _i32("stabilized_gates", read_slots, write_slots, entry_qstart)
    T = z.shape[0]
    if z.dtype != torch.float32 or z.stride(1) != 1 or max(i_off, f_off) + n_heads > z.shape[1]:
        raise KernelError("stabilized_gates: z float32 with a column per head at both offsets")
    if m_state.dtype != torch.float32 or not m_state.is_contiguous() or m_state.dim() != 2 or m_state.shape[1] != n_heads:
        raise KernelError("stabilized_gates: m_state float32 [slots, heads]")
    for t in (decay, in_weight, den_floor):
        if t.dtype != torch.float32 or tuple(t.shape) != (T, n_heads) or not t.is_contiguous():
            raise KernelError("stabilized_gates: outputs float32 [T, heads]")
    f = _fn("seqmix", "il_stabilized_gates", [_c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                              _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(z), z.stride(0), i_off, f_off, cap, _ptr(m_state), m_state.stride(0), _ptr(read_slots), _ptr(write_slots),
             _ptr(entry_qstart), _ptr(decay), _ptr(in_weight), _ptr(den_floor), n_heads, n_entries, first_entry, T, _stream()),
           "stabilized_gates")


GATE_SIGMOID, GATE_SILU = 0, 1


def group_norm_gate(x: torch.Tensor, w: torch.Tensor, eps: float, gate: torch.Tensor, g_off: int, act: int, out: torch.Tensor,
                    group: int, den_floor: Optional[torch.Tensor] = None, x_scale: float = 1.0, den_eps: float = 0.0) -> None:
    """out[t,j] = x[t,j] / sqrt(mean of x^2 over j's group of `group` columns + eps) * w[j % len(w)] * act(gate[t, g_off+j]);
    x float32 [T,n], gate float32 or bfloat16 (a view with a row stride), out float32 or bfloat16 [T,n].
    With `den_floor` (float32 [T, groups]) x is [T, groups * (group + 1)], every group followed by its normaliser column c:
    the group is first multiplied by x_scale and divided by max(|x_scale * c|, den_floor[t, g]) + den_eps."""
    _need_cuda(x, w, gate, out, den_floor)
    T = x.shape[0]
    if den_floor is not None:
        n_groups = x.shape[1] // (group + 1)
        if (x.shape[1] != n_groups * (group + 1) or den_floor.dtype != torch.float32 or tuple(den_floor.shape) != (T, n_groups)
                or not den_floor.is_contiguous()):
            raise KernelError("group_norm_gate: with a denominator x is [T, groups * (group + 1)] and den_floor float32 [T, groups]")
        n = n_groups * group
        if x.dtype != torch.float32 or x.stride(1) != 1 or out.stride(1) != 1 or gate.stride(1) != 1 or tuple(out.shape) != (T, n):
            raise KernelError("group_norm_gate: x float32, out [T, groups * group]")
        if g_off + n > gate.shape[1] or not w.is_contiguous():
            raise KernelError("group_norm_gate: the gate must cover the row")
        f = _fn("seqmix", "il_group_norm_gate_den", [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_float, _c_void_p, _c_int, _c_int,
                                                     _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_float,
                                                     _c_float, _c_void_p])
        _check(f(_ptr(x), x.stride(0), _ptr(w), kind_of(w.dtype), w.numel(), eps, _ptr(gate), kind_of(gate.dtype), gate.stride(0), g_off,
                 act, _ptr(out), kind_of(out.dtype), out.stride(0), group, n_groups, T, _ptr(den_floor), x_scale, den_eps, _stream()),
               "group_norm_gate")
        return
    n = x.shape[1]
    if x.dtype != torch.float32 or x.stride(1) != 1 or out.stride(1) != 1 or gate.stride(1) != 1 or tuple(out.shape) != (T, n):
        raise KernelError("group_norm_gate: x float32 [T,n], out [T,n]")
    if n % group or g_off + n > gate.shape[1] or not w.is_contiguous():
        raise KernelError("group_norm_gate: groups must divide the row, the gate must cover it")
    f = _fn("seqmix", "il_group_norm_gate", [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_float, _c_void_p, _c_int, _c_int, _c_int,
                                             _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), kind_of(w.dtype), w.numel(), eps, _ptr(gate), kind_of(gate.dtype), gate.stride(0), g_off,
             act, _ptr(out), kind_of(out.dtype), out.stride(0), group, n // group, T, _stream()), "group_norm_gate")


def head_gate(y: torch.Tensor, head_dim: int, gate: Optional[torch.Tensor], g_off: int, out: torch.Tensor, n_heads: int, vdim: int) -> None:
    """out[t, h*vdim + c] = y[t, h*head_dim + c] * sigmoid(gate[t, g_off + h]) for c < vdim: one gate per head, and heads that
    were padded to head_dim columns come out packed (`gate` None: only that)."""
    _need_cuda(y, gate, out)
    T = y.shape[0]
    if y.dtype != out.dtype or y.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("head_gate: one dtype, contiguous rows")
    if gate is not None and (gate.dtype != y.dtype or gate.stride(1) != 1 or g_off + n_heads > gate.shape[1]):
        raise KernelError("head_gate: the gate has y's dtype and one column per head")
    if y.shape[1] != n_heads * head_dim or tuple(out.shape) != (T, n_heads * vdim):
        raise KernelError("head_gate: shapes")
    f = _fn("seqmix", "il_head_gate", [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int,
                                       _c_int, _c_void_p])
    _check(f(_ptr(y), kind_of(y.dtype), y.stride(0), head_dim, _ptr(gate), 0 if gate is None else gate.stride(0), g_off, _ptr(out),
             out.stride(0), n_heads, vdim, T, _stream()), "head_gate")


def scaled_sum(a: torch.Tensor, sa: float, b: torch.Tensor, sb: float, out: torch.Tensor) -> None:
    """out = sa * a + sb * b, summed in float32; three contiguous tensors of one shape and dtype (out may be a or b)."""
    _need_cuda(a, b, out)
    if a.shape != b.shape or a.shape != out.shape or a.dtype != b.dtype or a.dtype != out.dtype:
        raise KernelError("scaled_sum: one shape and dtype")
    _contig("a", a), _contig("b", b), _contig("out", out)
    f = _fn("seqmix", "il_scaled_sum", [_c_void_p, _c_float, _c_void_p, _c_float, _c_void_p, _c_int, _c_ll, _c_void_p])
    _check(f(_ptr(a), sa, _ptr(b), sb, _ptr(out), kind_of(out.dtype), out.numel(), _stream()), "scaled_sum")


def softcap(y: torch.Tensor, cap: float) -> None:
    """y = cap * tanh(y / cap) in place, float32."""
    _need_cuda(y)
    if y.dtype != torch.float32 or not y.is_contiguous():
        raise KernelError("softcap: contiguous float32")
    f = _fn("seqmix", "il_softcap", [_c_void_p, _c_float, _c_ll, _c_void_p])
    _check(f(_ptr(y), cap, y.numel(), _stream()), "softcap")
