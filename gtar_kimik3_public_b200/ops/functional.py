"""Python faces of the kernels: argument checks, then one call into the kernel library.

Every function works on CUDA tensors on the current stream and allocates at most its own
output.  Shapes follow the packed ("varlen") convention of the step function: activations are
``[n_tokens, width]`` with the tokens of all sequences of a step one after another.
"""

from __future__ import annotations

import functools
from dataclasses import dataclass

import torch

from .library import KernelError, call, dtype_code, ptr, require_device, stream_ptr


def _check(tensor: torch.Tensor, name: str, dtype=None, dims: int | None = None) -> None:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if dims is not None and tensor.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got shape {tuple(tensor.shape)}")


@dataclass
class PagedKV:
    """One layer's keys and values in pages, and the table that maps a sequence's pages.

    ``k``, ``v``: ``[n_pages, n_kv_heads, page_size, head_dim]``; ``block_table``:
    ``[n_slots, max_pages]`` int32, entry ``[slot, i]`` = page that holds positions
    ``i*page_size .. (i+1)*page_size-1`` of the sequence in ``slot``.
    """

    k: torch.Tensor
    v: torch.Tensor
    block_table: torch.Tensor
    work: "DecodeWork | None" = None  # what decode attention keeps between launches; the cache group owns it

    @property
    def page_size(self) -> int:
        return self.k.shape[2]

    @property
    def max_pages(self) -> int:
        return self.block_table.shape[1]


class DecodeWork:
    """Scratch memory that decode attention keeps between launches, one per cache group (its layers run one after
    another on one stream): the partial results of sequences whose pages are shared by several blocks, and a ticket
    counter per (sequence, kv head), zero between launches (the kernel sets back what it counts up).  Buffers that
    are outgrown stay alive: a captured graph may still name them."""

    MIN_FLOATS, MIN_PAIRS = 1 << 18, 1024  # the least that is asked of the allocator, so that growth is rare

    def __init__(self, device: torch.device):
        self.device = device
        self.part: torch.Tensor | None = None
        self.tickets: torch.Tensor | None = None
        self.outgrown: list[torch.Tensor] = []

    def get(self, n_floats: int, n_pairs: int) -> tuple[torch.Tensor, torch.Tensor]:
        if self.part is None or self.part.numel() < n_floats:
            if self.part is not None:
                self.outgrown.append(self.part)
            self.part = torch.empty((max(n_floats, self.MIN_FLOATS),), dtype=torch.float32, device=self.device)
        if self.tickets is None or self.tickets.numel() < n_pairs:
            if self.tickets is not None:
                self.outgrown.append(self.tickets)
            self.tickets = torch.zeros((max(n_pairs, self.MIN_PAIRS),), dtype=torch.int32, device=self.device)
        return self.part, self.tickets


def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[t] = table[ids[t]]`` widened to float32 (the residual stream's type)."""
    require_device(table.device)
    _check(table, "table", dims=2)
    _check(ids, "ids", torch.int32, 1)
    n, hidden = ids.shape[0], table.shape[1]
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _check(out, "out", torch.float32, 2)
    call("gk_embed_rows", ptr(table), dtype_code(table.dtype), ptr(ids), ptr(out), n, hidden, stream_ptr())
    return out


def add_rmsnorm(
    h: torch.Tensor,
    delta: torch.Tensor | None,
    weight: torch.Tensor,
    eps: float,
    out_dtype: torch.dtype,
    rows: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """``h += delta`` (in place, skipped when ``delta`` is None), then RMSNorm of ``h`` times ``weight``.

    With ``rows`` (int32 indices) only those rows are normalised and ``h`` is not written: the
    sum ``h + delta`` of such a row is formed on the fly.
    """
    require_device(h.device)
    _check(h, "h", torch.float32, 2)
    _check(weight, "weight", dims=1)
    hidden = h.shape[1]
    if weight.shape[0] != hidden:
        raise KernelError(f"norm weight has {weight.shape[0]} entries for rows of {hidden}")
    delta_code = 0
    if delta is not None:
        _check(delta, "delta", dims=2)
        if delta.shape != h.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match h {tuple(h.shape)}")
        delta_code = dtype_code(delta.dtype)
    n_out = h.shape[0]
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        n_out = rows.shape[0]
    if out is None:
        out = torch.empty((n_out, hidden), dtype=out_dtype, device=h.device)
    _check(out, "out", out_dtype, 2)
    call(
        "gk_add_rmsnorm", ptr(h), ptr(delta), delta_code, ptr(weight), dtype_code(weight.dtype), ptr(out),
        dtype_code(out_dtype), ptr(rows), n_out, hidden, float(eps), stream_ptr(),
    )
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, interleaved: bool = False) -> torch.Tensor:
    """``silu(gate) * up`` for rows packed as ``[gate (I) | up (I)]``, or with ``interleaved`` as
    ``g0 u0 g1 u1 ...``."""
    require_device(gate_up.device)
    _check(gate_up, "gate_up", dims=2)
    n, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("gate_up rows must hold gate and up halves of equal width")
    inter = two_i // 2
    if out is None:
        out = torch.empty((n, inter), dtype=gate_up.dtype, device=gate_up.device)
    _check(out, "out", gate_up.dtype, 2)
    call("gk_swiglu", ptr(gate_up), ptr(out), dtype_code(gate_up.dtype), n, inter, int(interleaved), stream_ptr())
    return out


def qk_norm_rope_write(
    qkv: torch.Tensor,
    n_q: int,
    n_kv: int,
    head_dim: int,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    cos: torch.Tensor | None,
    sin: torch.Tensor | None,
    tok_pos: torch.Tensor,
    tok_seq: torch.Tensor,
    slots: torch.Tensor,
    kv: PagedKV,
    max_position: int,
    q_out: torch.Tensor | None = None,
    write_kv: bool = True,
) -> torch.Tensor:
    """Per-head RMSNorm of q and k, rotation by position, and the write of k and v into the pages.

    ``qkv``: ``[n_tokens, (n_q + 2 n_kv) * head_dim]``.  Returns the finished queries
    ``[n_tokens, n_q, head_dim]``.  ``max_position`` is the largest entry of ``tok_pos`` (known on
    the host) and is checked against the rotary table.  ``write_kv=False`` leaves the pages alone
    (a layer that attends over keys and values written by another layer).
    """
    require_device(qkv.device)
    _check(qkv, "qkv", dims=2)
    n = qkv.shape[0]
    if qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError(f"qkv rows are {qkv.shape[1]} wide, expected {(n_q + 2 * n_kv) * head_dim}")
    cache_dtype = qkv.dtype
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    _check(kv.block_table, "block_table", torch.int32, 2)
    _check(kv.k, "k pages", cache_dtype, 4)
    _check(kv.v, "v pages", cache_dtype, 4)
    if kv.k.shape[1] != n_kv or kv.k.shape[3] != head_dim or kv.v.shape != kv.k.shape:
        raise KernelError(f"pages {tuple(kv.k.shape)} do not fit n_kv={n_kv}, head_dim={head_dim}")
    use_norm = q_weight is not None
    weight_code = 0
    if use_norm:
        _check(q_weight, "q_weight", dims=1)
        _check(k_weight, "k_weight", q_weight.dtype, 1)
        if q_weight.shape[0] != head_dim or k_weight.shape[0] != head_dim:
            raise KernelError("q/k norm weights must have head_dim entries")
        weight_code = dtype_code(q_weight.dtype)
    table_positions = 0
    if cos is not None:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rotary tables must be [positions, head_dim / 2]")
        table_positions = cos.shape[0]
    if q_out is None:
        q_out = torch.empty((n, n_q, head_dim), dtype=cache_dtype, device=qkv.device)
    _check(q_out, "q_out", cache_dtype, 3)
    call(
        "gk_qk_norm_rope_write", ptr(qkv), dtype_code(qkv.dtype), ptr(q_weight), ptr(k_weight), weight_code, ptr(cos),
        ptr(sin), table_positions, ptr(tok_pos), ptr(tok_seq), ptr(slots), ptr(kv.block_table), ptr(q_out),
        ptr(kv.k) if write_kv else None, ptr(kv.v) if write_kv else None, n, n_q, n_kv, head_dim, kv.max_pages, kv.page_size, float(eps), int(use_norm), int(max_position),
        stream_ptr(),
    )
    return q_out


# Tiles of 128 x 256 from which the q|k|v product does its output stage itself.  Below, the library product and the
# stage as a kernel of its own are faster (1,024 tokens x 4,096 columns = 128 tiles: 16.2 against 17.7 us; 2,048
# tokens = 256 tiles: 26.7 against 25.9): the persistent kernel leaves SMs idle and its last tile's stage exposed.
QKV_FUSED_FROM_TILES = 200


def qkv_fused_ok(x: torch.Tensor, weight: torch.Tensor, head_dim: int, kv: PagedKV) -> bool:
    """Whether the q|k|v projection of this step can do the attention input stage in its epilogue:
    bfloat16, enough tokens for the many-token orientation and its wide tiles, head size 64 or 128."""
    m, k = x.shape
    n = weight.shape[0]
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and kv.k.dtype == torch.bfloat16
            and m > SKINNY_M and k % 8 == 0 and head_dim in (64, 128)
            and n >= PREFILL_BN and -(-m // 128) * -(-n // PREFILL_BN) >= QKV_FUSED_FROM_TILES)


def gemm_tc_qkv(
    x: torch.Tensor,
    weight: torch.Tensor,
    n_q: int,
    n_kv: int,
    head_dim: int,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    cos: torch.Tensor | None,
    sin: torch.Tensor | None,
    tok_pos: torch.Tensor,
    tok_seq: torch.Tensor,
    slots: torch.Tensor,
    kv: PagedKV,
    max_position: int,
    write_kv: bool = True,
) -> torch.Tensor:
    """``x @ weight.T`` for the packed q|k|v weight with per-head q/k RMSNorm, rotation and the write of
    k and v into the pages done in the product's epilogue.  Returns the queries ``[n_tokens, n_q, head_dim]``."""
    require_device(x.device)
    _check(x, "x", torch.bfloat16, 2)
    _check(weight, "weight", torch.bfloat16, 2)
    n, k = x.shape
    if weight.shape != ((n_q + 2 * n_kv) * head_dim, k):
        raise KernelError(f"weight is {tuple(weight.shape)}, expected {((n_q + 2 * n_kv) * head_dim, k)}")
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    _check(kv.k, "k pages", torch.bfloat16, 4)
    _check(kv.v, "v pages", torch.bfloat16, 4)
    if kv.k.shape[1] != n_kv or kv.k.shape[3] != head_dim:
        raise KernelError(f"pages {tuple(kv.k.shape)} do not fit n_kv={n_kv}, head_dim={head_dim}")
    use_norm = q_weight is not None
    weight_code = 0
    if use_norm:
        _check(q_weight, "q_weight", dims=1)
        _check(k_weight, "k_weight", q_weight.dtype, 1)
        weight_code = dtype_code(q_weight.dtype)
    table_positions = 0
    if cos is not None:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        table_positions = cos.shape[0]
    q_out = torch.empty((n, n_q, head_dim), dtype=torch.bfloat16, device=x.device)
    call(
        "gk_gemm_bf16_tc_qkv", ptr(x), n, ptr(weight), k, n_q, n_kv, head_dim, ptr(q_weight), ptr(k_weight), weight_code,
        int(use_norm), float(eps), ptr(cos), ptr(sin), table_positions, int(max_position), ptr(tok_pos), ptr(tok_seq),
        ptr(slots), ptr(kv.block_table), kv.max_pages, kv.page_size, ptr(q_out), ptr(kv.k) if write_kv else None,
        ptr(kv.v) if write_kv else None, ptr(error_flag(x.device)), stream_ptr(),
    )
    return q_out


def linear_f32(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.float32,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T`` on the FP32 pipes: ``weight`` float32 ``[N, K]``, ``x`` float32 or bfloat16 ``[M, K]``."""
    require_device(x.device)
    _check(x, "x", dims=2)
    _check(weight, "weight", torch.float32, 2)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"x is [{m}, {k}] but weight is {tuple(weight.shape)}")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    _check(out, "out", out_dtype, 2)
    call("gk_gemm_f32", ptr(x), dtype_code(x.dtype), ptr(weight), ptr(out), dtype_code(out_dtype), m, n, k, k, k, n,
         stream_ptr())
    return out


def attention_exact(
    q: torch.Tensor,
    kv: PagedKV,
    tok_pos: torch.Tensor,
    tok_seq: torch.Tensor,
    slots: torch.Tensor,
    scale: float,
    window: int = 0,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Causal grouped-query attention of ``q [n_tokens, n_q, d]`` over the pages (exact kernel)."""
    require_device(q.device)
    _check(q, "q", dims=3)
    n, n_q, d = q.shape
    _check(kv.k, "k pages", q.dtype, 4)
    _check(kv.v, "v pages", q.dtype, 4)
    n_kv = kv.k.shape[1]
    if kv.k.shape[3] != d:
        raise KernelError(f"pages have head_dim {kv.k.shape[3]}, queries {d}")
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    if out is None:
        out = torch.empty_like(q)
    call(
        "gk_attention_exact", ptr(q), ptr(kv.k), ptr(kv.v), ptr(out), dtype_code(q.dtype), ptr(tok_pos), ptr(tok_seq),
        ptr(slots), ptr(kv.block_table), n, n_q, n_kv, d, kv.max_pages, kv.page_size, float(scale), int(window),
        stream_ptr(),
    )
    return out


_error_flags: dict[int, torch.Tensor] = {}


def error_flag(device: torch.device) -> torch.Tensor:
    """The device int that kernels with bounded waits set when a wait gives up (0 = all well)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _error_flags:
        _error_flags[index] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[index]


def check_kernel_errors(device: torch.device | str = "cuda:0") -> None:
    """Raises if a kernel gave up a wait since the last check (synchronises the device)."""
    flag = error_flag(torch.device(device))
    code = int(flag.item())
    if code:
        flag.zero_()
        raise KernelError(f"a kernel gave up waiting on a barrier (code {code}); its output is not valid")


EPI_STORE, EPI_SWIGLU_A, EPI_SWIGLU_B = 0, 1, 2
SKINNY_M = 64  # up to this many tokens the weights take the MMA's 128 rows (swap-AB)


SPLIT_TARGET_BLOCKS = 128
PREFILL_BN = 256  # 128 x 256 tiles, walked by one persistent block per SM
SCRATCH_SPLITS_FROM = 17
SKINNY_BN_MAX = 64
SPLIT_MIN_K_BLOCKS = 4


_sm_counts: dict[int, int] = {}


def sm_count(device: torch.device | None = None) -> int:
    """Multiprocessors of the device (asked once per device)."""
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def split_k_for(m: int, n: int, k: int) -> int:
    """How many blocks share the K range of one output tile of a skinny product (m <= SKINNY_M).
    More blocks stream weights from more SMs: about 64 blocks in all, at least four k-blocks of 64
    each, and 1, 2, 4 or 8 ways (the blocks of a tile form one cluster)."""
    if m > SKINNY_M:
        return 1
    tiles = -(-n // 128) * -(-m // min(SKINNY_BN_MAX, 16 if m <= 16 else 32 if m <= 32 else 64))
    by_blocks = SPLIT_TARGET_BLOCKS // tiles
    if tiles * 8 <= SPLIT_TARGET_BLOCKS + 32:
        by_blocks = 8  # 17 to 20 tiles: eight ways (up to 160 blocks) beat four (2,560 rows of 9,728: 14.0 against 17.2 us)
    limit = min(by_blocks, (k // 64) // SPLIT_MIN_K_BLOCKS, 8)
    return 8 if limit >= 8 else 4 if limit >= 4 else 2 if limit >= 2 else 1


def set_pdl(on: bool) -> bool:
    """Switches programmatic dependent launch for all later kernel launches; returns the old setting."""
    from .library import library

    return bool(library().gk_set_pdl(int(on)))


GEMV_MAX_TOKENS = 16
GEMV_MAX_TOKENS_SHORT_K = 32  # with the activations of all tokens in registers (see gemv_suits)


def gemv_max_rows(device: torch.device) -> int:
    """Most weight rows ``gemv`` takes: one block per SM, each with up to eight groups of eight rows."""
    return sm_count(device) * 64



def set_gemm_pairs(mode: int) -> int:
    """How many-token products with wide tiles are run: 1 as pairs of blocks on one 256 x 256 tile (tcgen05
    cta_group::2), 0 as single blocks on 128 x 256 tiles, 2 (the default) pairs where the product is large
    enough for them to be the faster choice.  Returns the old setting."""
    from .library import library

    return int(library().gk_set_gemm_pairs(int(mode)))


def gemv_suits(m: int, n: int, k: int, device: torch.device) -> bool:
    """Whether ``gemv`` is the kernel for ``[m, k] @ [n, k].T``: few tokens, few enough weight rows, and
    activations that fit in shared memory beside a block's weights (it takes longer K too, in rounds, but
    there the tensor-memory product is the better choice).  17 to 32 tokens only where the activations of
    all of them stay in registers: K of 257 to 1,024 and a block's weights in shared memory at once."""
    if n > gemv_max_rows(device):
        return False
    if m <= GEMV_MAX_TOKENS:
        rows = 8 if m <= 8 else 16
        return k <= 1024 or rows * k * 2 <= 96 * 1024
    if m <= GEMV_MAX_TOKENS_SHORT_K:
        per_warp = -(-(-(-k // 32)) // 8)  # 32-wide chunks of K a warp takes per group of eight weight rows
        groups = -(-n // 8)
        per_block = -(-groups // min(groups, gemv_max_rows(device) // 64))
        return 2 <= per_warp <= 4 and per_block * per_warp <= 24
    return False


def gemv(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, swiglu: bool = False,
         out: torch.Tensor | None = None) -> torch.Tensor:
    """``x [M, K] @ weight[N, K].T`` for up to 16 tokens (32 where ``gemv_suits`` says so): weights go from memory straight into registers and
    through ``mma.sync`` with 32-bit accumulation; made for the latency of a decode step, where a projection
    is a few megabytes of weights and next to no arithmetic.  ``swiglu`` as in ``gemm_tc``."""
    require_device(x.device)
    _check(x, "x", torch.bfloat16, 2)
    _check(weight, "weight", torch.bfloat16, 2)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"x is {tuple(x.shape)} but weight is {tuple(weight.shape)}")
    if m > GEMV_MAX_TOKENS_SHORT_K:
        raise KernelError(f"gemv takes up to {GEMV_MAX_TOKENS_SHORT_K} tokens, got {m}")
    if swiglu and n % 2:
        raise KernelError("the SwiGLU epilogue needs an even number of weight rows")
    n_out = n // 2 if swiglu else n
    if out is None:
        out = torch.empty((m, n_out), dtype=out_dtype, device=x.device)
    _check(out, "out", out_dtype, 2)
    if tuple(out.shape) != (m, n_out):
        raise KernelError(f"out has shape {tuple(out.shape)}, expected {(m, n_out)}")
    call("gk_gemv_bf16", ptr(weight), n, k, k, ptr(x), m, k, ptr(out), dtype_code(out_dtype), int(swiglu), stream_ptr())
    return out


def gemv_normed_suits(m: int, n: int, k: int, device: torch.device) -> bool:
    """Whether ``gemv_stream`` can form its activations as the RMSNorm of a 32-bit stream itself: up to 16 tokens whose
    rows (up to 1,024 long) a block's threads hold whole, and a block's weights in shared memory at once."""
    if m > GEMV_MAX_TOKENS or k > 1024 or k % 8 or n > gemv_max_rows(device):
        return False
    per_warp = -(-(-(-k // 32)) // 8)
    groups = -(-n // 8)
    per_block = -(-groups // min(groups, gemv_max_rows(device) // 64))
    return per_block * per_warp <= 24


def gemv_stream(weight: torch.Tensor, x: torch.Tensor | None = None, norm: tuple | None = None, resid: torch.Tensor | None = None,
                swiglu: bool = False, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor | None:
    """The few-token product with the residual stream at either end.

    ``norm = (h, norm_weight, eps)``: the activations are the RMSNorm of the rows of the 32-bit stream ``h [tokens, k]``,
    formed inside the kernel (no norm kernel in front).  ``resid``: the 32-bit stream ``[tokens, n]`` that the result,
    rounded to bfloat16 as a projection's output is, is added to in place (no add in the norm kernel behind); nothing
    is returned then.  Otherwise as ``gemv``."""
    require_device(weight.device)
    _check(weight, "weight", torch.bfloat16, 2)
    n, k = weight.shape
    if norm is not None:
        h, norm_weight, eps = norm
        _check(h, "h", torch.float32, 2)
        _check(norm_weight, "norm weight", dims=1)
        m = h.shape[0]
        if h.shape[1] != k or norm_weight.shape[0] != k:
            raise KernelError(f"the stream is {tuple(h.shape)} and the norm's weight {tuple(norm_weight.shape)} for rows of {k}")
        if not gemv_normed_suits(m, n, k, weight.device):
            raise KernelError(f"the norm on load does not take {m} tokens of {k} with {n} weight rows")
    else:
        _check(x, "x", torch.bfloat16, 2)
        m = x.shape[0]
        if x.shape[1] != k:
            raise KernelError(f"x is {tuple(x.shape)} but weight is {tuple(weight.shape)}")
        h, norm_weight, eps = None, None, 1.0
    out = None
    if resid is not None:
        _check(resid, "resid", torch.float32, 2)
        if tuple(resid.shape) != (m, n) or swiglu:
            raise KernelError(f"the residual stream must be {(m, n)} (and no SwiGLU), got {tuple(resid.shape)}")
    else:
        out = torch.empty((m, n // 2 if swiglu else n), dtype=out_dtype, device=weight.device)
    call("gk_gemv_bf16_stream", ptr(weight), n, k, k, ptr(x), m, k, ptr(out), dtype_code(out_dtype), int(swiglu), ptr(h), k,
         ptr(norm_weight), int(norm_weight is not None and norm_weight.dtype == torch.bfloat16), float(eps), ptr(resid), n, stream_ptr())
    return out


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, swiglu: bool = False,
            splits: int = 1, out: torch.Tensor | None = None) -> torch.Tensor:
    """``x [M, K] @ weight[N, K].T`` in bfloat16 on the tcgen05 tensor cores, float32 accumulation.

    ``swiglu=True``: the rows of ``weight`` alternate gate, up, gate, up, ...; the result is
    ``silu(gate) * up`` of width ``N / 2``.  ``splits > 1`` shares the K range of every output tile
    among 2, 4 or 8 blocks (a skinny product then streams weights from more SMs); the blocks form a
    cluster and add their partial tiles through distributed shared memory in a fixed order.
    """
    require_device(x.device)
    _check(x, "x", torch.bfloat16, 2)
    _check(weight, "weight", torch.bfloat16, 2)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"x is {tuple(x.shape)} but weight is {tuple(weight.shape)}")
    if swiglu and n % 2:
        raise KernelError("the SwiGLU epilogue needs an even number of weight rows")
    n_out = n // 2 if swiglu else n
    if out is None:
        out = torch.empty((m, n_out), dtype=out_dtype, device=x.device)
    _check(out, "out", out_dtype, 2)
    if tuple(out.shape) != (m, n_out):
        raise KernelError(f"out has shape {tuple(out.shape)}, expected {(m, n_out)}")
    flag = error_flag(x.device)
    if m <= SKINNY_M:
        bn = 16 if m <= 16 else 32 if m <= 32 else 64
        bn = min(bn, SKINNY_BN_MAX)
        call("gk_gemm_bf16_tc", ptr(weight), n, k, ptr(x), m, k, k, ptr(out), dtype_code(out_dtype), 1, n_out,
             EPI_SWIGLU_A if swiglu else EPI_STORE, bn, splits, 1, 0, ptr(flag), stream_ptr())
    else:
        wide = n >= PREFILL_BN and -(-m // 128) * -(-n // PREFILL_BN) >= 120  # enough wide tiles to fill the GPU
        bn = PREFILL_BN if wide else 128 if n >= 128 else 64 if n >= 64 else 32 if n >= 32 else 16
        call("gk_gemm_bf16_tc", ptr(x), m, k, ptr(weight), n, k, k, ptr(out), dtype_code(out_dtype), n_out, 1,
             EPI_SWIGLU_B if swiglu else EPI_STORE, bn, splits, 0, 1, ptr(flag), stream_ptr())
    return out


@functools.lru_cache(maxsize=None)
def decode_cluster_places(head_dim: int, sm_count: int) -> tuple[int, int, int, int]:
    """How many clusters of 1, 2, 4 and 8 blocks of the decode attention kernel the device holds at once.  Asked of the
    device where there is one (clusters are placed inside a GPC, so eight-block clusters fill fewer of the SMs' places
    than single blocks do); two blocks an SM otherwise."""
    if torch.cuda.is_available():
        from .library import library

        got = [library().gk_attention_decode_resident_clusters(int(head_dim), c) for c in (1, 2, 4, 8)]
        if all(g > 0 for g in got):
            return tuple(got)
    return tuple(2 * sm_count // c for c in (1, 2, 4, 8))


@functools.lru_cache(maxsize=4096)
def decode_splits(n_seqs: int, n_kv: int, max_kv_len: int, page_size: int, sm_count: int,
                  cluster_places: tuple[int, int, int, int] | None = None) -> int:
    """How many blocks share a sequence's pages in decode attention.

    Two blocks fit an SM.  With few (sequence, kv head) pairs and a long context, as many splits as fill those
    places go through scratch and a second kernel.  Otherwise 1, 2, 4 or 8 splits merge inside the kernel (a
    cluster per pair, which then does the q/k preparation too), and the number is the one with the lowest
    estimate of  waves of clusters x (pages a block streams + 8 pages' worth of time for what a block does
    besides); ``cluster_places`` says how many clusters of 1, 2, 4 and 8 blocks run at once (default: two blocks
    an SM, whatever the cluster).  It agrees with step times measured at batch 1 to 64 with 2,048-token contexts;
    against the old "fill the places once" rule it gains 7 to 13% at batch 12, 40 and 48 (clusters of three place
    badly: two splits are faster; 320 or 384 pairs are better cut in two than run as one and a bit waves)."""
    pairs = max(1, n_seqs * n_kv)
    pages = max(1, -(-max_kv_len // page_size))
    places = 2 * sm_count
    fill = max(1, min(places // pairs, pages, 64))
    # (one and two sequences of 8,192 tokens are faster as clusters of eight, 0.83 and 0.91 ms a step against 0.85 and 0.98
    # through scratch; of 16,384 tokens slower, 1.18 and 1.45 against 1.03 and 1.32)
    if fill >= SCRATCH_SPLITS_FROM and max_kv_len >= 12288:
        return fill
    if cluster_places is None:
        cluster_places = tuple(places // c for c in (1, 2, 4, 8))
    at_once = dict(zip((1, 2, 4, 8), cluster_places))

    def estimate(splits: int) -> float:
        # clusters of eight that have to share SMs cost more besides their pages than the eight say, the more of the SMs
        # hold two of their blocks (four sequences of 2,048 tokens: 0.73 ms a step with four splits, 0.76 with eight; three
        # sequences: 0.70 with four, 0.65 with eight; one and two sequences are faster with eight)
        besides = 8.0
        if splits == 8 and pairs * splits > sm_count:
            besides = 13.0 if pairs * splits > 1.5 * sm_count else 10.0
        return -(-pairs // max(1, at_once[splits])) * (pages / splits + besides)

    return min((s for s in (1, 2, 4, 8) if s <= pages), key=lambda s: (estimate(s), s))


def decode_flat_wins(n_seqs: int, n_kv: int, kv_len: int, page_size: int, sm_count: int,
                     cluster_places: tuple[int, int, int, int] | None, flat_places: int) -> bool:
    """Whether dealing the step's pages out evenly among all blocks is expected to beat the best equal cut.

    The evenly dealt kernel costs some 7 us more than the equal cut where that fits the device (partial results
    through scratch, a ticket per part, a merge by whoever comes last), so it is chosen where the equal cut fits
    badly.  Measured, 28 layers of the 0.6B sizes, ms a step with the equal cut against dealt evenly:

    * blocks that come in two waves of which the second is thin: contexts of 2,048, 40 sequences (320 pairs on 296
      places) 2.86 / 2.57, 44: 2.88 / 2.78, but 48: 2.89 / 2.91, 52: 3.00 / 3.05, 56: 3.13 / 3.21, 60: 3.17 / 3.33; contexts
      of 512, 40: 1.57 / 1.53; of 1,024, 40: 2.05 / 1.91 but 56: 2.16 / 2.26;
    * three and more waves of clusters: contexts of 4,096, 40 sequences (five waves of clusters of four) 4.13 / 3.90; of
      8,192, 40: 6.67 / 6.61;
    * whole sequences a block that fill little more than half of the places and are long: 20 sequences of 4,096
      2.57 / 2.34, of 8,192 4.06 / 3.70, but of 2,048 1.66 / 1.70; 24 of 2,048 1.71 / 1.83, of 4,096 2.72 / 2.70;
    * clusters of eight that share SMs on long contexts: 32,768 tokens, 3 sequences 2.66 / 2.42, 4: 3.17 / 2.92; 16,384, 4:
      2.09 / 2.05 but 3: 1.34 / 1.64, 6 (cut in four): 2.37 / 2.63; 8,192, 4: 1.19 / 1.45.

    Elsewhere the equal cut is ahead: 8 sequences of 2,048 tokens 0.82 / 1.1, 12: 1.11 / 1.21, 16: 1.25 / 1.5, 32: 1.98 / 2.2,
    64: 3.26 / 3.5; 12 of 8,192 (cut in two): 2.33 / 2.48."""
    splits = decode_splits(n_seqs, n_kv, kv_len, page_size, sm_count, cluster_places)
    if splits > 8:
        return False
    pairs = max(1, n_seqs * n_kv)
    pages = max(1, -(-kv_len // page_size))
    if cluster_places is None:
        cluster_places = tuple(2 * sm_count // c for c in (1, 2, 4, 8))
    at_once = max(1, dict(zip((1, 2, 4, 8), cluster_places))[splits])
    waves = -(-pairs // at_once)
    fill = pairs / (waves * at_once)
    per_block = pairs * pages / flat_places  # pages a block streams when they are dealt evenly
    if waves == 1:
        if splits == 8 and pairs * 8 > sm_count:
            # the more of the SMs hold two blocks of a cluster of eight, the sooner
            return per_block >= (24 if pairs * 8 > 1.5 * sm_count else 30)
        return splits == 1 and fill < 0.66 and per_block >= 28
    return fill < (0.62 if waves == 2 else 0.92)


def attention_decode(
    q: torch.Tensor,
    kv: PagedKV,
    kv_len: torch.Tensor,
    slots: torch.Tensor,
    scale: float,
    window: int = 0,
    n_splits: int = 1,
    out: torch.Tensor | None = None,
    use_scratch: bool = False,
) -> torch.Tensor:
    """Attention of one new token per sequence (``q [n_seqs, n_q, d]`` bfloat16, ``d`` 64 or 128) over
    the pages; ``kv_len[i]`` counts the sequence's cached tokens including the new one.  Up to eight
    splits merge inside one kernel (a cluster per sequence and kv head); more, or ``use_scratch``, go
    through scratch memory allocated here and a second kernel."""
    require_device(q.device)
    _check(q, "q", torch.bfloat16, 3)
    n, n_q, d = q.shape
    _check(kv.k, "k pages", torch.bfloat16, 4)
    _check(kv.v, "v pages", torch.bfloat16, 4)
    _check(kv_len, "kv_len", torch.int32, 1)
    _check(slots, "slots", torch.int32, 1)
    if kv_len.shape[0] != n or slots.shape[0] != n:
        raise KernelError("kv_len and slots need one entry per sequence")
    n_kv = kv.k.shape[1]
    if kv.k.shape[3] != d:
        raise KernelError(f"pages have head_dim {kv.k.shape[3]}, queries {d}")
    if out is None:
        out = torch.empty_like(q)
    part_o = part_ml = None
    if n_splits > 8 or (n_splits > 1 and use_scratch):
        part_o = torch.empty((n * n_q * n_splits * d,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * n_q * n_splits * 2,), dtype=torch.float32, device=q.device)
    call(
        "gk_attention_decode_bf16", ptr(q), ptr(kv.k), ptr(kv.v), ptr(out), ptr(part_o), ptr(part_ml), ptr(kv_len),
        ptr(slots), ptr(kv.block_table), n, n_q, n_kv, d, kv.max_pages, kv.page_size, float(scale), int(window),
        int(n_splits), stream_ptr(),
    )
    return out


def attention_decode_fused(
    qkv: torch.Tensor,
    n_q: int,
    n_kv: int,
    head_dim: int,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    cos: torch.Tensor | None,
    sin: torch.Tensor | None,
    kv: PagedKV,
    kv_len: torch.Tensor,
    slots: torch.Tensor,
    max_position: int,
    scale: float,
    window: int = 0,
    n_splits: int = 1,
    write_kv: bool = True,
) -> torch.Tensor:
    """Decode attention straight from the packed projection of the new tokens: per-head q/k RMSNorm,
    rotation, the write of the new key and value into the pages and the attention itself in one kernel
    (bfloat16, head size 64 or 128, at most 8 splits).  Returns ``[n_seqs, n_q, head_dim]``."""
    require_device(qkv.device)
    _check(qkv, "qkv", torch.bfloat16, 2)
    n = qkv.shape[0]
    if qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError(f"qkv rows are {qkv.shape[1]} wide, expected {(n_q + 2 * n_kv) * head_dim}")
    _check(kv.k, "k pages", torch.bfloat16, 4)
    _check(kv.v, "v pages", torch.bfloat16, 4)
    _check(kv_len, "kv_len", torch.int32, 1)
    _check(slots, "slots", torch.int32, 1)
    if kv.k.shape[1] != n_kv or kv.k.shape[3] != head_dim:
        raise KernelError(f"pages {tuple(kv.k.shape)} do not fit n_kv={n_kv}, head_dim={head_dim}")
    if n_splits > 8:
        raise KernelError("the fused decode attention takes at most 8 splits")
    use_norm = q_weight is not None
    weight_code = 0
    if use_norm:
        _check(q_weight, "q_weight", dims=1)
        _check(k_weight, "k_weight", q_weight.dtype, 1)
        weight_code = dtype_code(q_weight.dtype)
    table_positions = 0
    if cos is not None:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rotary tables must be [positions, head_dim / 2]")
        table_positions = cos.shape[0]
    out = torch.empty((n, n_q, head_dim), dtype=torch.bfloat16, device=qkv.device)
    call(
        "gk_attention_decode_fused_bf16", ptr(qkv), ptr(q_weight), ptr(k_weight), weight_code, int(use_norm), float(eps),
        ptr(cos), ptr(sin), table_positions, int(max_position), int(write_kv), ptr(kv.k), ptr(kv.v), ptr(out), None, None,
        ptr(kv_len), ptr(slots), ptr(kv.block_table), n, n_q, n_kv, head_dim, kv.max_pages, kv.page_size, float(scale),
        int(window), int(n_splits), stream_ptr(),
    )
    return out


@functools.lru_cache(maxsize=None)
def decode_flat_places(head_dim: int, sm_count: int) -> int:
    """How many blocks of the evenly dealt decode attention kernel the device holds at once: the most pieces that
    the step's pages are cut into.  Asked of the device where there is one; two blocks an SM otherwise."""
    if torch.cuda.is_available():
        from .library import library

        got = library().gk_attention_decode_flat_resident_blocks(int(head_dim))
        if got > 0:
            return got
    return 2 * sm_count


def attention_decode_flat(
    q: torch.Tensor | None,
    qkv: torch.Tensor | None,
    n_q: int,
    n_kv: int,
    head_dim: int,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    cos: torch.Tensor | None,
    sin: torch.Tensor | None,
    kv: PagedKV,
    kv_len: torch.Tensor,
    slots: torch.Tensor,
    max_position: int,
    scale: float,
    window: int = 0,
    n_blocks: int = 0,
    write_kv: bool = True,
) -> torch.Tensor:
    """Decode attention with the pages of all sequences dealt out evenly among ``n_blocks`` blocks (0: as many
    as the device holds at once), whatever the sequences' lengths.  Either ``q [n_seqs, n_q, head_dim]`` (keys and
    values are in the pages) or the packed projection ``qkv [n_seqs, (n_q + 2 n_kv) * head_dim]`` of the new tokens,
    which the kernel then norms, rotates and writes itself as ``attention_decode_fused`` does.  Returns
    ``[n_seqs, n_q, head_dim]`` bfloat16."""
    if (q is None) == (qkv is None):
        raise KernelError("either q or qkv")
    given = q if qkv is None else qkv
    require_device(given.device)
    if qkv is None:
        _check(q, "q", torch.bfloat16, 3)
        if q.shape[1] != n_q or q.shape[2] != head_dim:
            raise KernelError(f"q is {tuple(q.shape)}, expected [n, {n_q}, {head_dim}]")
    else:
        _check(qkv, "qkv", torch.bfloat16, 2)
        if qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
            raise KernelError(f"qkv rows are {qkv.shape[1]} wide, expected {(n_q + 2 * n_kv) * head_dim}")
    n = given.shape[0]
    _check(kv.k, "k pages", torch.bfloat16, 4)
    _check(kv.v, "v pages", torch.bfloat16, 4)
    _check(kv_len, "kv_len", torch.int32, 1)
    _check(slots, "slots", torch.int32, 1)
    if kv_len.shape[0] != n or slots.shape[0] != n:
        raise KernelError("kv_len and slots need one entry per sequence")
    if kv.k.shape[1] != n_kv or kv.k.shape[3] != head_dim:
        raise KernelError(f"pages {tuple(kv.k.shape)} do not fit n_kv={n_kv}, head_dim={head_dim}")
    use_norm = qkv is not None and q_weight is not None
    weight_code = 0
    if use_norm:
        _check(q_weight, "q_weight", dims=1)
        _check(k_weight, "k_weight", q_weight.dtype, 1)
        weight_code = dtype_code(q_weight.dtype)
    table_positions = 0
    if qkv is not None and cos is not None:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rotary tables must be [positions, head_dim / 2]")
        table_positions = cos.shape[0]
    else:
        cos = sin = None
    if n_blocks <= 0:
        n_blocks = decode_flat_places(head_dim, sm_count(given.device))
    work = kv.work if kv.work is not None else DecodeWork(given.device)
    part, tickets = work.get((n_blocks + n * n_kv) * (n_q // n_kv) * (head_dim + 2), n * n_kv)
    out = torch.empty((n, n_q, head_dim), dtype=torch.bfloat16, device=given.device)
    call(
        "gk_attention_decode_flat_bf16", ptr(q), ptr(qkv), ptr(q_weight) if use_norm else None,
        ptr(k_weight) if use_norm else None, weight_code, int(use_norm), float(eps), ptr(cos), ptr(sin), table_positions,
        int(max_position), int(write_kv), ptr(kv.k), ptr(kv.v), ptr(out), ptr(part), ptr(tickets), ptr(kv_len), ptr(slots),
        ptr(kv.block_table), n, n_q, n_kv, head_dim, kv.max_pages, kv.page_size, float(scale), int(window), int(n_blocks),
        stream_ptr(),
    )
    return out


def attention_prefill(
    q: torch.Tensor,
    kv: PagedKV,
    cu_q: torch.Tensor,
    kv_len: torch.Tensor,
    slots: torch.Tensor,
    max_q_len: int,
    scale: float,
    window: int = 0,
    out: torch.Tensor | None = None,
    tensor_cores: str = "auto",
) -> torch.Tensor:
    """Causal attention of the packed new tokens ``q [n_tokens, n_q, d]`` (bfloat16, ``d`` 64 or 128) of
    ``n_seqs`` sequences over the pages.  Sequence ``i`` owns tokens ``cu_q[i] .. cu_q[i+1]-1``, which
    are its last positions: ``kv_len[i]`` counts its cached tokens including them.  ``tensor_cores``:
    ``"tcgen05"`` (head size 128 only), ``"mma"`` (the warp-level kernel), or ``"auto"``."""
    require_device(q.device)
    _check(q, "q", torch.bfloat16, 3)
    n, n_q, d = q.shape
    _check(kv.k, "k pages", torch.bfloat16, 4)
    _check(kv.v, "v pages", torch.bfloat16, 4)
    for name, t in (("cu_q", cu_q), ("kv_len", kv_len), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    n_seqs = kv_len.shape[0]
    if cu_q.shape[0] != n_seqs + 1 or slots.shape[0] != n_seqs:
        raise KernelError("cu_q needs n_seqs + 1 entries, slots and kv_len n_seqs")
    n_kv = kv.k.shape[1]
    if kv.k.shape[3] != d:
        raise KernelError(f"pages have head_dim {kv.k.shape[3]}, queries {d}")
    if out is None:
        out = torch.empty_like(q)
    if tensor_cores not in ("auto", "tcgen05", "mma"):
        raise KernelError(f"tensor_cores must be auto, tcgen05 or mma, got {tensor_cores!r}")
    if tensor_cores == "tcgen05" and d != 128:
        raise KernelError("the tcgen05 prefill attention takes head size 128 only")
    if tensor_cores == "tcgen05" or (tensor_cores == "auto" and d == 128):
        call(
            "gk_attention_prefill_tc_tokens_bf16", ptr(q), ptr(kv.k), ptr(kv.v), ptr(out), ptr(cu_q), ptr(kv_len), ptr(slots),
            ptr(kv.block_table), n_seqs, int(max_q_len), n_q, n_kv, d, kv.max_pages, kv.page_size, kv.k.shape[0],
            float(scale), int(window), ptr(error_flag(q.device)), stream_ptr(), int(q.shape[0]),
        )
        return out
    call(
        "gk_attention_prefill_bf16", ptr(q), ptr(kv.k), ptr(kv.v), ptr(out), ptr(cu_q), ptr(kv_len), ptr(slots),
        ptr(kv.block_table), n_seqs, int(max_q_len), n_q, n_kv, d, kv.max_pages, kv.page_size, float(scale), int(window),
        stream_ptr(),
    )
    return out


def set_attention_prefill_keys(keys: int) -> int:
    """Keys per step of the tcgen05 prefill attention: 128 (the default: one block per SM, two score buffers,
    two threads a row, a heavy and a light query tile per block) or 64 (two blocks per SM, one query tile
    each).  Returns the old setting."""
    from .library import library

    return int(library().gk_set_attention_prefill_keys(int(keys)))


def set_attention_prefill_stay(mode: int) -> int:
    """Whether the tcgen05 prefill attention (128 keys a step) runs as blocks that stay, one an SM, and take query tiles
    from the launch's list with the next tile's queries and first scores under the tile in hand: 1 = always, 2 (the
    default) = where the launch has more tiles than the device SMs, 0 = never (a block a tile).  Returns the old setting."""
    from .library import library

    return int(library().gk_set_attention_prefill_stay(int(mode)))


def set_attention_prefill_one_tile(mode: int) -> int:
    """How the tcgen05 prefill attention (128 keys a step) deals out its query tiles: 1 (the default) = a tile a
    block with the heaviest first, 0 = a heavy and a light tile a block.  Returns the old setting."""
    from .library import library

    return int(library().gk_set_attention_prefill_one_tile(int(mode)))


def row_parts(n_rows: int, vocab: int, device: torch.device) -> int:
    """Blocks that share a row of logits in the token choice: about eight blocks per multiprocessor in all, slices
    of at least 4,096 entries, at most 64 a row."""
    return max(1, min(8 * sm_count(device) // max(n_rows, 1), vocab // 4096, 64))


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Index of the largest logit of each row (lowest index on ties), int32."""
    require_device(logits.device)
    _check(logits, "logits", torch.float32, 2)
    n, vocab = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(out, "out", torch.int32, 1)
    # few rows of a wide vocabulary: several blocks share a row so that the scan uses the whole GPU
    parts = row_parts(n, vocab, logits.device)
    scratch = torch.empty((n * parts * 2,), dtype=torch.int32, device=logits.device) if parts > 1 else None
    call("gk_argmax", ptr(logits), vocab, n, vocab, ptr(out), parts, ptr(scratch), stream_ptr())
    return out


def sample(
    logits: torch.Tensor,
    temperature: float,
    top_k: int,
    seed: int,
    request_ids: torch.Tensor,
    steps: torch.Tensor,
    advance_steps: bool = False,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Temperature (+ top-k) sampling by the Gumbel-max rule with counter-based uniforms.

    Row ``r`` draws with the key ``(seed, request_ids[r], steps[r])``; with ``advance_steps`` the
    kernel adds one to ``steps[r]`` afterwards, so a loop replayed from a CUDA graph needs no host
    work between tokens.
    """
    require_device(logits.device)
    _check(logits, "logits", torch.float32, 2)
    n, vocab = logits.shape
    _check(request_ids, "request_ids", torch.int32, 1)
    _check(steps, "steps", torch.int32, 1)
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(out, "out", torch.int32, 1)
    # as for argmax: several blocks share a row; eight bytes of scratch per row for the top-k thresholds (four
    # used) and eight per row and part for the parts' results
    parts = row_parts(n, vocab, logits.device)
    scratch = torch.empty((2 * ((n + 1) // 2) + 2 * n * parts,), dtype=torch.int32, device=logits.device)
    call(
        "gk_sample", ptr(logits), vocab, n, vocab, float(temperature), int(top_k or 0), int(seed) & (2**64 - 1),
        ptr(request_ids), ptr(steps), int(advance_steps), ptr(out), parts, ptr(scratch), stream_ptr(),
    )
    return out


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``x @ weight.T`` for bfloat16 operands with 32-bit accumulation (library matrix product,
    as the reference's nn.Linear under autocast is: src/engine.py:35)."""
    require_device(x.device)
    _check(x, "x", torch.bfloat16, 2)
    _check(weight, "weight", torch.bfloat16, 2)
    if weight.shape[1] != x.shape[1]:
        raise KernelError(f"x is {tuple(x.shape)} but weight is {tuple(weight.shape)}")
    y = torch.mm(x, weight.t())
    return y if out_dtype == torch.bfloat16 else y.to(out_dtype)


# ------------------------------------------------------------------ a run of layers of a decode step as one kernel
DECODE_LAYERS_MAX_SEQS = 8


def decode_layers_work_sizes(n_seqs: int, hidden: int, n_q: int, n_kv: int, head_dim: int, inter: int, max_kv_len: int,
                             page_size: int) -> tuple[int, int] | None:
    """(floats of partial results, 32-bit words of counters) that ``decode_layers`` needs for these sizes, or None if
    the kernel does not take them (the library's message says why: ``library().gk_last_error()``)."""
    import ctypes

    from .library import library

    out = (ctypes.c_longlong * 2)()
    status = library().gk_decode_layers_plan(n_seqs, hidden, n_q, n_kv, head_dim, inter, max_kv_len, page_size, out)
    return (int(out[0]), int(out[1])) if status == 0 else None


def decode_layers(layer_table: torch.Tensor, n_layers: int, h: torch.Tensor, n_q: int, n_kv: int, head_dim: int, inter: int,
                  qkv: torch.Tensor, att: torch.Tensor, act: torch.Tensor, part: torch.Tensor, words: torch.Tensor,
                  kv_len: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, max_kv_len: int,
                  cos: torch.Tensor | None, sin: torch.Tensor | None, norm_bf16: bool, qk_bf16: bool, scale: float,
                  stamps: torch.Tensor | None = None) -> None:
    """Runs ``n_layers`` pre-norm layers (RMSNorm, grouped-query attention with per-head q/k norm and rotation over
    the paged cache, RMSNorm, SwiGLU) of a decode step on the stream ``h [n_seqs, hidden]`` (float32, updated in
    place) as one persistent kernel.  ``layer_table``: the layers' pointers and constants as the kernel's records (96
    bytes each, see ``models/persistent_decode.py``); ``qkv``, ``att``, ``act``, ``part``, ``words``: work areas
    (``words`` zero before the first call; the kernel leaves it zero).  ``stamps`` (int64 ``[blocks, 5 n_layers, 2]``,
    for measurements): every block's clock readings, in nanoseconds, at its arrival at and release from each barrier."""
    require_device(h.device)
    _check(h, "h", torch.float32, 2)
    _check(layer_table, "layer_table", torch.uint8, 1)
    n_seqs, hidden = h.shape
    if layer_table.shape[0] < 96 * n_layers:
        raise KernelError("the layer table is shorter than its layers")
    for name, t, dtype in (("qkv", qkv, torch.bfloat16), ("att", att, torch.bfloat16), ("act", act, torch.bfloat16),
                           ("part", part, torch.float32), ("words", words, torch.int32), ("kv_len", kv_len, torch.int32),
                           ("slots", slots, torch.int32)):
        _check(t, name, dtype)
    _check(block_table, "block_table", torch.int32, 2)
    if qkv.numel() < n_seqs * (n_q + 2 * n_kv) * head_dim or att.numel() < n_seqs * n_q * head_dim or act.numel() < n_seqs * inter:
        raise KernelError("a work area is smaller than the step needs")
    if words.numel() < 8 + n_seqs * n_kv or kv_len.shape[0] != n_seqs or slots.shape[0] != n_seqs:
        raise KernelError("counters, lengths and slots need one entry per sequence (and kv head)")
    table_positions = 0
    if cos is not None:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rotary tables must be [positions, head_dim / 2]")
        table_positions = cos.shape[0]
    call("gk_decode_layers", ptr(layer_table), n_layers, n_seqs, hidden, n_q, n_kv, head_dim, inter, ptr(h), ptr(qkv), ptr(att),
         ptr(act), ptr(part), part.numel(), ptr(words), ptr(kv_len), ptr(slots), ptr(block_table), block_table.shape[1],
         int(max_kv_len), ptr(cos), ptr(sin), table_positions, int(norm_bf16), int(qk_bf16), float(scale),
         ptr(error_flag(h.device)), ptr(stamps), stream_ptr())
