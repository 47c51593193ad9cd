"""Python faces of the CUDA kernels: they check tensors and launch on the
current CUDA stream.  Every function needs CUDA tensors; there is no CPU path."""
from __future__ import annotations

import torch

from . import library
from .library import KernelError, check

F32, BF16 = 0, 1


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {dtype}: the kernels take float32 and bfloat16")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors: torch.Tensor) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError("the kernels run on CUDA tensors only; there is no CPU fallback")


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


_SM_COUNT: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (the current one by default): launch heuristics size
    their grids by it instead of carrying one GPU's number."""
    index = torch.cuda.current_device() if device is None or torch.device(device).index is None else torch.device(device).index
    count = _SM_COUNT.get(index)
    if count is None:
        count = _SM_COUNT[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return count


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, copies: int = 1, scale: float = 1.0) -> torch.Tensor:
    """out[t] = float32(table[ids[t]]) * scale, ``copies`` times side by side; ids int32 [T], out float32 [T, copies * H]."""
    _need_cuda(table, ids, out)
    vocab, hidden = table.shape
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.is_contiguous()
    assert out.shape == (ids.shape[0], copies * hidden) and out.is_contiguous()
    lib = library.load()
    check(lib.lse_embedding_scaled(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), out.data_ptr(),
                                   ids.shape[0], hidden, vocab, int(copies), float(scale), _stream()), "embedding")
    return out


def _partials(tensor: torch.Tensor | None, rows: int, width: int):
    """(tensor, number of partial sums, elements between them) of a [rows, width] tensor or a
    float32 stack of partial sums [P, rows, width]."""
    if tensor is None:
        return None, 1, 0
    if tensor.dim() == 3:
        assert tensor.dtype == torch.float32 and tensor.shape[1:] == (rows, width) and tensor.is_contiguous()
        return tensor, tensor.shape[0], rows * width
    assert tensor.shape == (rows, width) and tensor.is_contiguous()
    return tensor, 1, 0


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: torch.Tensor | None = None, write_residual: bool = True) -> torch.Tensor:
    """residual (+= delta); out = rmsnorm(residual) * weight.

    residual float32 [T, H]; delta [T, H] float32/bfloat16, a float32 stack of partial sums
    [P, T, H] (added in index order), or None; weight float32 [H]; out [R, H]
    float32/bfloat16 where R = len(rows) when ``rows`` (int32 row indices into residual) is
    given, else T.  With ``rows`` the residual is left unchanged unless ``write_residual``.
    """
    _need_cuda(residual, delta, weight, out, rows)
    tokens, hidden = residual.shape
    assert residual.dtype == torch.float32 and weight.dtype == torch.float32 and weight.shape == (hidden,)
    assert residual.is_contiguous() and out.is_contiguous() and out.shape[-1] == hidden
    delta, n_partials, stride = _partials(delta, tokens, hidden)
    n_rows = out.shape[0]
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.shape[0] == n_rows
    else:
        assert n_rows == tokens
    lib = library.load()
    delta_code = dtype_code(delta.dtype) if delta is not None else dtype_code(out.dtype)
    check(lib.lse_add_rmsnorm(residual.data_ptr(), _ptr(delta), delta_code, n_partials, stride, weight.data_ptr(),
                              out.data_ptr(), dtype_code(out.dtype), _ptr(rows), n_rows, hidden,
                              float(eps), int(write_residual), tokens, _stream()), "add_rmsnorm")
    return out


def gemm_f32_nt(a: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ weight[N, K]^T (+ bias[N]) in true float32."""
    _need_cuda(a, weight, bias, out)
    m, k = a.shape
    n = weight.shape[0]
    assert a.dtype == weight.dtype == out.dtype == torch.float32
    assert weight.shape[1] == k and out.shape == (m, n)
    assert a.stride(1) == 1 and weight.stride(1) == 1 and out.stride(1) == 1
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.shape == (n,)
    lib = library.load()
    check(lib.lse_gemm_f32_nt(a.data_ptr(), weight.data_ptr(), _ptr(bias), out.data_ptr(), m, n, k,
                              a.stride(0), weight.stride(0), out.stride(0), 0, 0, _stream()), "gemm_f32_nt")
    return out


def gemm_f32_stack_ok(a: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether :func:`gemm_f32_stack` takes this product (few rows, k a multiple of 4, aligned rows)."""
    return bool(library.load().lse_gemm_f32_stack_ok(a.data_ptr(), weight.data_ptr(), a.shape[0], a.shape[1],
                                                     a.stride(0), weight.stride(0)))


def gemm_f32_stack(a: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """a @ weight^T in true float32 as a stack [P, M, N] of the sums over the k ranges that the product is
    always cut into: a block per range, so that a product of few rows has enough blocks to stream the weights.
    Added up in index order, starting from zero, the stack gives :func:`gemm_f32_nt`'s result bit for bit."""
    _need_cuda(a, weight)
    m, k = a.shape
    n = weight.shape[0]
    assert a.dtype == weight.dtype == torch.float32 and weight.shape[1] == k
    assert a.stride(1) == 1 and weight.stride(1) == 1
    lib = library.load()
    ranges = int(lib.lse_gemm_f32_ranges(k))
    out = torch.empty((ranges, m, n), dtype=torch.float32, device=a.device)
    check(lib.lse_gemm_f32_nt(a.data_ptr(), weight.data_ptr(), None, out.data_ptr(), m, n, k,
                              a.stride(0), weight.stride(0), out.stride(1), 1, out.stride(0), _stream()), "gemm_f32_stack")
    return out


def rope_kv_write(qkv: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor,
                  slot_mapping: torch.Tensor, inv_freq: torch.Tensor, q_out: torch.Tensor,
                  k_cache: torch.Tensor, v_cache: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                  pairing: int) -> None:
    """Bias, rotary encoding of queries and keys, and the write of keys and values
    into the paged cache (k_cache/v_cache: [pages, n_kv, page_size, head_dim]).
    ``qkv`` is [T, width] in the cache's dtype or in float32, or a float32 stack of
    partial sums [P, T, width]."""
    _need_cuda(qkv, bias, positions, slot_mapping, inv_freq, q_out, k_cache, v_cache)
    width = (n_q + 2 * n_kv) * head_dim
    tokens = qkv.shape[-2]
    if qkv.dim() == 3:
        qkv, n_partials, stride = _partials(qkv, tokens, width)
        row_stride = width
    else:
        assert qkv.shape[1] == width and qkv.stride(1) == 1
        n_partials, stride, row_stride = 1, 0, qkv.stride(0)
    assert positions.dtype == torch.int32 and slot_mapping.dtype == torch.int32
    assert positions.shape[0] >= tokens and slot_mapping.shape[0] >= tokens
    assert inv_freq.dtype == torch.float32 and inv_freq.shape == (head_dim // 2,)
    assert q_out.dtype == k_cache.dtype == v_cache.dtype
    assert q_out.is_contiguous() and q_out.shape == (tokens, n_q, head_dim)
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape[1] == n_kv and k_cache.shape[3] == head_dim and v_cache.shape == k_cache.shape
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.shape == (width,)
    lib = library.load()
    check(lib.lse_rope_kv_write(qkv.data_ptr(), dtype_code(qkv.dtype), n_partials, stride, _ptr(bias),
                                positions.data_ptr(), slot_mapping.data_ptr(), inv_freq.data_ptr(),
                                q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), dtype_code(q_out.dtype),
                                tokens, n_q, n_kv, head_dim, k_cache.shape[2], pairing, row_stride, k_cache.shape[0],
                                _stream()),
          "rope_kv_write")


GENERIC_SPLIT_MAX_ROWS = 64   # up to this many rows every chunk of keys of a row gets a block of its own


def paged_attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                            out: torch.Tensor, block_tables: torch.Tensor,
                            segment_of_token: torch.Tensor, positions: torch.Tensor, scale: float,
                            window: int = 0, split: bool | None = None) -> torch.Tensor:
    """Attention of every token of the step over its request's cached keys.

    q, out [T, n_q, D]; k_cache, v_cache [pages, n_kv, page_size, D];
    block_tables int32 [S, max_pages]; segment_of_token, positions int32 [T].
    A row's keys are summed in chunks of fixed size; ``split`` gives every chunk a block of its own
    (default: with few rows, where one block per row would leave the GPU idle).  The result does not
    depend on it, bit for bit.
    """
    _need_cuda(q, k_cache, v_cache, out, block_tables, segment_of_token, positions)
    tokens, n_q, head_dim = q.shape
    n_kv, page_size = k_cache.shape[1], k_cache.shape[2]
    if head_dim % 16 or head_dim > 256:
        raise KernelError(f"attention: head size {head_dim} is not a multiple of 16 up to 256")
    if n_q % n_kv:
        raise KernelError(f"attention: {n_q} query heads do not divide into {n_kv} groups")
    assert q.is_contiguous() and out.is_contiguous() and out.shape == q.shape
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.shape == k_cache.shape
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype
    assert block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.stride(1) == 1
    assert segment_of_token.dtype == torch.int32 and positions.dtype == torch.int32
    lib = library.load()
    partials, max_chunks = None, 0
    if split if split is not None else tokens <= GENERIC_SPLIT_MAX_ROWS:
        chunk = int(lib.lse_attention_generic_chunk())
        max_chunks = max(1, -(-(block_tables.stride(0) * page_size) // chunk))
        partials = torch.empty(tokens * n_q * max_chunks * (head_dim + 2), dtype=torch.float32, device=q.device)
    check(lib.lse_paged_attention_generic(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                          out.data_ptr(), dtype_code(q.dtype), block_tables.data_ptr(),
                                          block_tables.stride(0), segment_of_token.data_ptr(),
                                          positions.data_ptr(), tokens, n_q, n_kv, head_dim, page_size,
                                          float(scale), int(window), k_cache.shape[0], block_tables.shape[0],
                                          partials.data_ptr() if partials is not None else None, max_chunks,
                                          _stream()), "paged_attention_generic")
    return out


def attention_mma_supported(head_dim: int, n_q: int, n_kv: int, dtype: torch.dtype, window: int = 0) -> bool:
    """Whether the tensor-core attention kernels take this shape (bfloat16, head size 64 or 128,
    no window); other shapes run the general kernel."""
    if dtype != torch.bfloat16 or window > 0:
        return False
    return bool(library.load().lse_attention_mma_supported(head_dim, n_q, n_kv))


_DECODE_MAX_SPLITS = int(__import__("os").environ.get("LSE_DECODE_MAX_SPLITS", "8"))


_DECODE_MAX_SPLITS_LONG = 32    # the kernel's own limit


def decode_splits(tokens: int, n_q: int, n_kv: int, max_context: int | None, long_context: bool = False) -> int:
    """How many splits of the keys a decode launch uses: enough blocks to fill the GPU and a little
    more (a block that ends early makes room for the next kernel's blocks), at least one 16-key
    tile per warp and split.  (A block takes up to 8 query heads of a group.)"""
    base = tokens * n_kv * ((n_q // n_kv + 7) // 8)
    # about 1.4 blocks per SM (measured best from 12 to 64 rows on 148 SMs: 192 blocks beat 128 and 256); at most
    # 8 splits: one cluster adds them up.  Over long contexts (more than 8,192 keys) with so few rows that 8 splits
    # leave SMs without a block, more splits pay although the last-arriving block then adds them up through global
    # memory (one request of 30,000 keys: 1.60 against 2.05 ms a step; four: 1.87 against 2.13; at 8,192 keys: no gain).
    cap = _DECODE_MAX_SPLITS
    if long_context and 10 * base * cap < 7 * sm_count():
        cap = max(cap, _DECODE_MAX_SPLITS_LONG)
    splits = max(1, min(cap, ((sm_count() * 7 + 4) // 5) // base))
    if max_context is not None:
        splits = min(splits, max(1, -(-max_context // 64)))
    return splits


_ARRIVALS: dict = {}


def _arrival_counters(device, count: int) -> torch.Tensor:
    """Zeroed int32 counters that the split-KV kernel uses and leaves zero; kept per device
    so that a captured graph finds them at the same address."""
    held = _ARRIVALS.get(device)
    if held is None or held.numel() < count:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("arrival counters must exist before a stream is captured")
        held = torch.zeros(max(count, 4096), dtype=torch.int32, device=device)
        _ARRIVALS[device] = held
    return held


def paged_attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                           block_tables: torch.Tensor, segment_of_token: torch.Tensor, positions: torch.Tensor,
                           scale: float, num_splits: int, cluster: bool = True,
                           segment_start: torch.Tensor | None = None,
                           segment_first_position: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of single decoded tokens (one row per request) with the keys split over
    ``num_splits`` blocks; bfloat16, head size 64 or 128.  With ``segment_start`` (int32 [S + 1], a step that
    also holds prompt portions) the rows are those of the requests that bring exactly one token, wherever they
    lie among q's rows; the other rows of ``out`` are left alone.  With ``segment_first_position`` (int32 [S])
    the rows may be rows of prompt portions, several of a request: every row walks its keys on its own (for
    steps of few rows, where the prompt kernels would leave most of the GPU idle)."""
    _need_cuda(q, k_cache, v_cache, out, block_tables, segment_of_token, positions)
    tokens, n_q, head_dim = q.shape
    n_kv, page_size = k_cache.shape[1], k_cache.shape[2]
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert block_tables.dtype == torch.int32 and block_tables.stride(1) == 1
    if segment_start is not None:
        _need_cuda(segment_start)
        assert segment_start.dtype == torch.int32 and segment_start.shape[0] == block_tables.shape[0] + 1
        tokens = block_tables.shape[0]      # one block row per request of the step
    scratch = arrivals = None
    by_cluster = cluster and 1 < num_splits <= 8      # the splits add up through distributed shared memory
    if num_splits > 1 and not by_cluster:
        scratch = torch.empty(tokens * n_q * num_splits * (head_dim + 2), dtype=torch.float32, device=q.device)
        arrivals = _arrival_counters(q.device, tokens * n_kv * ((n_q // n_kv + 7) // 8))
    lib = library.load()
    check(lib.lse_paged_attention_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                         _ptr(scratch), _ptr(arrivals), int(by_cluster), block_tables.data_ptr(),
                                         block_tables.stride(0),
                                         segment_of_token.data_ptr(), positions.data_ptr(), tokens, n_q, n_kv,
                                         head_dim, page_size, float(scale), int(num_splits), k_cache.shape[0],
                                         block_tables.shape[0], _ptr(segment_start), _ptr(segment_first_position), _stream()),
          "paged_attention_decode")
    return out


def paged_attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                            block_tables: torch.Tensor, segment_start: torch.Tensor,
                            segment_first_position: torch.Tensor, scale: float, skip_single: bool = False,
                            max_portions: int = 0) -> torch.Tensor:
    """Attention of prompt portions (any mix of segment lengths): causal inside the portion,
    all earlier keys of the request before it; bfloat16, head size 64 or 128.

    segment_start int32 [S + 1]: first row of each segment; segment_first_position int32 [S].
    ``skip_single``: requests that bring exactly one token are left to :func:`paged_attention_decode`;
    ``max_portions`` (with it): at most so many requests bring more than one token (it sizes the grid).
    """
    _need_cuda(q, k_cache, v_cache, out, block_tables, segment_start, segment_first_position)
    tokens, n_q, head_dim = q.shape
    n_kv, page_size = k_cache.shape[1], k_cache.shape[2]
    segments = segment_first_position.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert block_tables.dtype == torch.int32 and block_tables.stride(1) == 1 and segment_start.shape[0] == segments + 1
    lib = library.load()
    check(lib.lse_paged_attention_prefill(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                          block_tables.data_ptr(), block_tables.stride(0), segment_start.data_ptr(),
                                          segment_first_position.data_ptr(), segments, tokens, n_q, n_kv, head_dim,
                                          page_size, float(scale), k_cache.shape[0], int(skip_single),
                                          int(max_portions) if skip_single else 0, _stream()),
          "paged_attention_prefill")
    return out


def attention_tc_supported(head_dim: int, n_q: int, n_kv: int, page_size: int, dtype: torch.dtype,
                           window: int = 0) -> bool:
    """Whether the tcgen05 prefill kernel takes this shape (bfloat16, head size 64 or 128, pages of
    8 to 128 keys that divide 128, no window)."""
    if dtype != torch.bfloat16 or window > 0:
        return False
    return bool(library.load().lse_attention_tc_supported(head_dim, n_q, n_kv, page_size))


def paged_attention_prefill_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                               block_tables: torch.Tensor, segment_start: torch.Tensor,
                               segment_first_position: torch.Tensor, scale: float, skip_single: bool = False,
                               max_portions: int = 0, share_keys: bool = True) -> torch.Tensor:
    """Attention of prompt portions on the 5th-generation tensor cores: the arguments and the
    result of :func:`paged_attention_prefill`; blocks of 128 rows of one head, keys in tiles of 128
    brought in by TMA page by page, scores and outputs accumulated in tensor memory.  In a launch with fewer
    blocks than the GPU has SMs several blocks share the keys of a tile of rows; ``share_keys=False`` keeps every
    tile in one block (for comparisons)."""
    _need_cuda(q, k_cache, v_cache, out, block_tables, segment_start, segment_first_position)
    tokens, n_q, head_dim = q.shape
    pages, n_kv, page_size = k_cache.shape[0], k_cache.shape[1], k_cache.shape[2]
    segments = segment_first_position.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert v_cache.shape == k_cache.shape and k_cache.shape[3] == head_dim
    assert block_tables.dtype == torch.int32 and block_tables.stride(1) == 1 and segment_start.shape[0] == segments + 1
    lib = library.load()
    scratch, counters = _attention_tc_scratch(q.device) if share_keys else (None, None)
    check(lib.lse_paged_attention_prefill_tc(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                             block_tables.data_ptr(), block_tables.stride(0), segment_start.data_ptr(),
                                             segment_first_position.data_ptr(), segments, tokens, pages, n_q, n_kv,
                                             head_dim, page_size, float(scale), int(skip_single),
                                             int(max_portions) if skip_single else 0, _ptr(scratch), _ptr(counters),
                                             counters.shape[0] if counters is not None else 0, _stream()),
          "paged_attention_prefill_tc")
    return out


_ATTENTION_TC_SCRATCH: dict = {}


def _attention_tc_scratch(device) -> tuple[torch.Tensor, torch.Tensor]:
    """Where the blocks of the tcgen05 prompt attention that share the keys of one tile of rows leave their parts
    (a launch with fewer blocks than SMs), and the arrival counters, which the kernel leaves at zero.  One pair per
    device, made at the first call (never inside a graph capture: a size class runs once before it is captured)."""
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    pair = _ATTENTION_TC_SCRATCH.get(index)
    if pair is None:
        slots = sm_count(index)
        floats = int(library.load().lse_attention_tc_scratch_floats())
        where = torch.device("cuda", index)
        pair = _ATTENTION_TC_SCRATCH[index] = (torch.empty(slots * floats, dtype=torch.float32, device=where),
                                               torch.zeros(slots, dtype=torch.int32, device=where))
    return pair


def attention_tc_status() -> int:
    """0 while no bounded wait of the tcgen05 attention kernel has given up (synchronises the device)."""
    return int(library.load().lse_attention_tc_status())


GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu": 2, "clamped_swish": 3}


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu", limit: float = 0.0) -> torch.Tensor:
    """out[t, i] = act(gate_i) * up_i; ``gate_up`` is [T, 2I] (the row is [gate (I) | up (I)]) or a
    float32 stack of partial sums [P, T, 2I]; ``activation``: "silu", "gelu_tanh" (the tanh form of GELU), "relu", or
    "clamped_swish": g = min(gate, limit), u = clamp(up, -limit, limit), out = g sigmoid(1.702 g) (u + 1)."""
    _need_cuda(gate_up, out)
    tokens, two_i = gate_up.shape[-2], gate_up.shape[-1]
    assert two_i % 2 == 0 and out.shape == (tokens, two_i // 2) and out.is_contiguous()
    gate_up, n_partials, stride = _partials(gate_up, tokens, two_i)
    lib = library.load()
    check(lib.lse_gated_act_mul_limit(gate_up.data_ptr(), dtype_code(gate_up.dtype), n_partials, stride, out.data_ptr(),
                                      dtype_code(out.dtype), tokens, two_i // 2, GATE_ACTIVATIONS[activation],
                                      float(limit), _stream()), "silu_mul")
    return out


GEMM_SKINNY_MAX_ROWS = 256      # rows of x the few-rows product takes
_GEMM_BLOCKS_PER_SM = 2     # two blocks of the few-rows product fit on an SM; LSE_GEMM_BLOCKS overrides the total
_GEMM_MAX_SPLITS = int(__import__("os").environ.get("LSE_GEMM_MAX_SPLITS", "16"))


def _gemm_target_blocks() -> int:
    override = __import__("os").environ.get("LSE_GEMM_BLOCKS")
    return int(override) if override else _GEMM_BLOCKS_PER_SM * sm_count()


def gemm_bf16_skinny_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the few-rows tensor-core product takes these operands."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[0] <= GEMM_SKINNY_MAX_ROWS
            and x.shape[1] % 8 == 0 and x.is_contiguous() and weight.is_contiguous()
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_bf16_skinny(x: torch.Tensor, weight: torch.Tensor, splits: int | None = None, stages: int = 6,
                     max_splits: int | None = None, block_n: int = 128) -> torch.Tensor:
    """Partial sums [P, M, N] (float32) of x[M, K] @ weight[N, K]^T for M <= 256, bfloat16 operands;
    the k range is cut into P splits so that enough blocks stream the weights."""
    _need_cuda(x, weight)
    m, k = x.shape
    n = weight.shape[0]
    if not gemm_bf16_skinny_ok(x, weight) or weight.shape[1] != k:
        raise KernelError("gemm_bf16_skinny: operands must be contiguous bfloat16, K a multiple of 8, at most 256 rows")
    lib = library.load()
    if splits is None:
        # about two blocks per SM (more of the weights are fetched ahead while earlier kernels run), but no
        # more splits than keep the partial sums (4 bytes per row, column and split) well below the weight bytes
        n_tiles = -(-n // block_n)
        splits = 1 if n_tiles >= sm_count() else max(1, min(-(-k // 128), _gemm_target_blocks() // n_tiles,
                                                             max(1, k // (4 * m)), max_splits or _GEMM_MAX_SPLITS))
    splits = lib.lse_gemm_bf16_skinny_splits(k, int(splits))
    out = torch.empty((splits, m, n), dtype=torch.float32, device=x.device)
    check(lib.lse_gemm_bf16_skinny(x.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k, splits, int(stages),
                                   int(block_n), _stream()), "gemm_bf16_skinny")
    return out


def gemm_bf16_skinny_test_hooks(spin_limit: int = 0, withhold: bool = False) -> None:
    """For tests of the bounded waits: ``spin_limit`` iterations before a wait gives up (0: the default),
    ``withhold``: every block leaves out its last weight tile, so that a wait runs out."""
    torch.cuda.synchronize()
    check(library.load().lse_gemm_bf16_skinny_test_hooks(int(spin_limit), int(bool(withhold))), "gemm test hooks")


def gemm_bf16_skinny_status() -> int:
    """0 unless a bounded wait inside the kernel has given up (synchronises the device)."""
    return int(library.load().lse_gemm_bf16_skinny_status())


def kernel_status_async(host_words: torch.Tensor) -> None:
    """Queue, on the current stream, copies of the status words of the kernels with bounded waits (the
    few-rows product, the tcgen05 prompt attention) into ``host_words`` (pinned int32 [2]).  Once the
    stream has got there, a non-zero word says that a wait gave up: that block wrote nothing, and
    what the step computed is not to be used."""
    assert host_words.dtype == torch.int32 and host_words.numel() >= 2 and host_words.is_pinned()
    lib = library.load()
    stream = _stream()
    if lib.lse_gemm_bf16_skinny_status_async(host_words.data_ptr(), stream) != 0 or \
            lib.lse_attention_tc_status_async(host_words.data_ptr() + 4, stream) != 0:
        raise KernelError("the kernels' status words could not be read")


def kernel_status_reset() -> None:
    """Clear both status words (after a failure has been reported)."""
    lib = library.load()
    lib.lse_gemm_bf16_skinny_status_reset()
    lib.lse_attention_tc_status_reset()
    for _, counters in _ATTENTION_TC_SCRATCH.values():   # a block that gave up may have left its arrival uncounted
        counters.zero_()


def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = index of the first largest value of logits[r] (float32 [R, V])."""
    _need_cuda(logits, out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    rows, vocab = logits.shape
    lib = library.load()
    check(lib.lse_argmax(logits.data_ptr(), logits.stride(0), rows, vocab, out.data_ptr(), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, seed: torch.Tensor,
           counter: torch.Tensor, scratch: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Temperature / top-p sampling of one token per row (rows with temperature <= 0 take the argmax).

    temperature, top_p float32 [R]; seed, counter int64 [R]; scratch float32 with
    at least R * V values; out int32 [R].
    """
    _need_cuda(logits, temperature, top_p, seed, counter, scratch, out)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32
    assert seed.dtype == torch.int64 and counter.dtype == torch.int64
    assert scratch.dtype == torch.float32 and scratch.numel() >= rows * vocab and scratch.is_contiguous()
    lib = library.load()
    check(lib.lse_sample(logits.data_ptr(), logits.stride(0), rows, vocab, temperature.data_ptr(),
                         top_p.data_ptr(), seed.data_ptr(), counter.data_ptr(), scratch.data_ptr(),
                         out.data_ptr(), _stream()), "sample")
    return out


# ------------------------------------------------------------------ residual kept in several copies
def streams_update_rmsnorm(streams: torch.Tensor, n_streams: int, delta: torch.Tensor | None,
                           scale: torch.Tensor | None, mult: float, mix: torch.Tensor | None,
                           write_weights: torch.Tensor | None, read_weights: torch.Tensor | None,
                           weight: torch.Tensor, eps: float, out: torch.Tensor, rows: torch.Tensor | None = None,
                           write_back: bool = True) -> torch.Tensor:
    """The pending branch output goes into the copies of the residual, then the next branch's input is read and normed.

    streams float32 [T, S * H] (S copies of width H side by side); delta [T, H], a float32 stack [P, T, H], or None;
    X'[t] = sum_s mix[s, t] X[s] + write_weights[t] * mult * scale * delta  (mix None: identity; write None: ones;
    scale float32 [H] or None); u = sum_t read_weights[t] X'[t] (None: ones); out = u / sqrt(mean(u^2) + eps) * weight.
    ``rows``: int32 row numbers (out has one row each); ``write_back``: store X'."""
    _need_cuda(streams, delta, scale, mix, write_weights, read_weights, weight, out, rows)
    tokens = streams.shape[0]
    hidden = streams.shape[1] // n_streams
    assert streams.dtype == torch.float32 and streams.is_contiguous() and streams.shape[1] == n_streams * hidden
    assert weight.dtype == torch.float32 and weight.shape == (hidden,) and out.is_contiguous() and out.shape[1] == hidden
    for table, count in ((scale, hidden), (mix, n_streams * n_streams), (write_weights, n_streams), (read_weights, n_streams)):
        assert table is None or (table.dtype == torch.float32 and table.numel() == count and table.is_contiguous())
    delta, n_partials, stride = _partials(delta, tokens, hidden)
    n_rows = out.shape[0]
    assert (rows is None and n_rows == tokens) or (rows is not None and rows.dtype == torch.int32 and rows.shape[0] == n_rows)
    lib = library.load()
    delta_code = dtype_code(delta.dtype) if delta is not None else F32
    check(lib.lse_streams_update_rmsnorm(streams.data_ptr(), _ptr(delta), delta_code, n_partials, stride, _ptr(scale),
                                         float(mult), _ptr(mix), _ptr(write_weights), _ptr(read_weights),
                                         weight.data_ptr(), out.data_ptr(), dtype_code(out.dtype), _ptr(rows), n_rows,
                                         int(n_streams), hidden, float(eps), int(write_back), tokens, _stream()),
          "streams_update_rmsnorm")
    return out


def _projection(proj: torch.Tensor):
    """(tensor, dtype code, partial sums, elements between them, elements between rows) of a projection's result:
    [T, N] in float32 or bfloat16 (rows may be strided) or a float32 stack of partial sums [P, T, N]."""
    if proj.dim() == 3:
        assert proj.dtype == torch.float32 and proj.is_contiguous()
        return proj, F32, proj.shape[0], proj.shape[1] * proj.shape[2], proj.shape[2]
    assert proj.dim() == 2 and proj.stride(1) == 1
    return proj, dtype_code(proj.dtype), 1, 0, proj.stride(0)


# ------------------------------------------------------------------ linear attention with a decay
LINEAR_ATTENTION_ACTIVATIONS = {"none": 0, "silu": 1}


LINEAR_ATTENTION_CHUNK = 64          # rows of a chunk when a step's rows are scanned in chunks
LINEAR_ATTENTION_CHUNKED_FROM = 128  # rows of a step from which they are


def linear_attention_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, decay: torch.Tensor,
                          state: torch.Tensor, segment_start: torch.Tensor, segment_slot: torch.Tensor,
                          out: torch.Tensor, heads: int, dim: int, vdim: int, activation: str = "silu",
                          chunked: bool | None = None) -> torch.Tensor:
    """S = decay_h S + k v^T, o = S^T q over the rows of every request of the step, in order, from and into
    ``state`` float32 [slots, heads, dim, vdim].  q, k, v are act(columns of ``proj``) (head h of q at
    q_off + h * dim and so on); out float32 [T, heads * vdim].  ``chunked`` (default: from
    ``LINEAR_ATTENTION_CHUNKED_FROM`` rows on): the rows of a request are cut into chunks that are scanned side by
    side (each chunk's own state from zero, the states carried from chunk to chunk, then the outputs from each
    chunk's starting state); the result differs from the row-by-row scan by rounding only."""
    _need_cuda(proj, decay, state, segment_start, segment_slot, out)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens = proj.shape[-2]
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (heads, dim, vdim)
    assert decay.dtype == torch.float32 and decay.shape == (heads,)
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == (tokens, heads * vdim)
    assert segment_start.dtype == torch.int32 and segment_slot.dtype == torch.int32
    segments = segment_slot.shape[0]
    assert segment_start.shape[0] == segments + 1
    lib = library.load()
    chunk_rows, chunk_state, max_chunks = 0, None, 0
    if chunked if chunked is not None else tokens >= LINEAR_ATTENTION_CHUNKED_FROM:
        chunk_rows = LINEAR_ATTENTION_CHUNK
        max_chunks = tokens // chunk_rows + segments
        chunk_state = torch.empty((max_chunks, heads, dim, vdim), dtype=torch.float32, device=out.device)
    check(lib.lse_linear_attention_scan(proj.data_ptr(), code, n_partials, stride, ld, q_off, k_off, v_off,
                                        decay.data_ptr(), state.data_ptr(), segment_start.data_ptr(),
                                        segment_slot.data_ptr(), out.data_ptr(), segments, heads, dim, vdim,
                                        LINEAR_ATTENTION_ACTIVATIONS[activation], state.shape[0], chunk_rows,
                                        _ptr(chunk_state), max_chunks, _stream()),
          "linear_attention_scan")
    return out


def gated_rmsnorm(values: torch.Tensor, proj: torch.Tensor, g_off: int, weight: torch.Tensor, eps: float,
                  out: torch.Tensor, segment_of_token: torch.Tensor | None = None) -> torch.Tensor:
    """out = values / sqrt(mean(values^2) + eps) * weight * sigmoid(gate); values float32 [T, N]; the gate is columns
    g_off .. g_off + N of ``proj``."""
    _need_cuda(values, proj, weight, out, segment_of_token)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens, n = values.shape
    assert values.dtype == torch.float32 and values.is_contiguous() and weight.dtype == torch.float32 and weight.shape == (n,)
    assert out.shape == (tokens, n) and out.is_contiguous()
    lib = library.load()
    check(lib.lse_gated_rmsnorm(values.data_ptr(), proj.data_ptr(), code, n_partials, stride, ld, g_off,
                                weight.data_ptr(), out.data_ptr(), dtype_code(out.dtype), tokens, n, float(eps),
                                _ptr(segment_of_token), _stream()), "gated_rmsnorm")
    return out


# ------------------------------------------------------------------ attention over a cached latent
def latent_prepare(proj: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor, eps: float, *,
                   q_off: int = 0, q_rank: int = 0, q_norm: torch.Tensor | None = None,
                   q_latent: torch.Tensor | None = None, kv_off: int = -1, rank: int = 0,
                   kv_norm: torch.Tensor | None = None, rot: int = 0, rot_dims: int = 0,
                   freq: torch.Tensor | None = None, rot_factor: float = 1.0, cache: torch.Tensor | None = None,
                   g_off: int = -1, heads: int = 0, gate: torch.Tensor | None = None) -> None:
    """Per row of the step, from the fused down-projection ``proj``: the normed query latent (columns q_off .. +q_rank,
    into ``q_latent`` [T, q_rank]); the normed key/value latent (kv_off .. +rank) and the rotated shared key part (the
    next ``rot`` columns, the first ``rot_dims`` of them rotated) into the token's row of ``cache`` [pages, page_size,
    rank + rot]; sigmoid of the gate columns (g_off .. +heads) into ``gate`` float32 [T, heads].  Each piece is optional."""
    _need_cuda(proj, positions, slot_mapping, q_norm, q_latent, kv_norm, freq, cache, gate)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens = proj.shape[-2]
    out_dtype = q_latent.dtype if q_latent is not None else cache.dtype if cache is not None else torch.float32
    if q_rank:
        assert q_latent.shape == (tokens, q_rank) and q_latent.is_contiguous() and q_norm.dtype == torch.float32
    num_slots = 0
    if kv_off >= 0:
        assert cache.is_contiguous() and cache.shape[-1] == rank + rot and cache.dtype == out_dtype
        assert kv_norm.dtype == torch.float32 and kv_norm.shape == (rank,)
        assert freq.dtype == torch.float64 and freq.shape[0] >= rot_dims // 2
        num_slots = cache.shape[0] * cache.shape[1]
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.shape == (tokens, heads) and gate.is_contiguous()
    lib = library.load()
    check(lib.lse_latent_prepare(proj.data_ptr(), code, n_partials, stride, ld, q_off, q_rank, _ptr(q_norm),
                                 _ptr(q_latent), kv_off, rank, _ptr(kv_norm), rot, rot_dims, _ptr(freq),
                                 float(rot_factor), positions.data_ptr(), slot_mapping.data_ptr(), _ptr(cache),
                                 dtype_code(out_dtype), g_off, heads, _ptr(gate), float(eps), tokens, num_slots,
                                 proj.shape[-1], _stream()), "latent_prepare")


def latent_query(proj: torch.Tensor, q_off: int, heads: int, dim: int, rot: int, rot_dims: int, freq: torch.Tensor,
                 rot_factor: float, positions: torch.Tensor, segment_of_token: torch.Tensor, q_plain: torch.Tensor,
                 q_wide: torch.Tensor, at: int) -> None:
    """Head h's query is columns q_off + h * (dim + rot) .. of ``proj``: its first ``dim`` values go to ``q_plain``
    [T, heads, dim], its last ``rot`` values, rotated, to ``q_wide`` [T, heads, wide] from column ``at``."""
    _need_cuda(proj, freq, positions, segment_of_token, q_plain, q_wide)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens = proj.shape[-2]
    assert q_plain.shape == (tokens, heads, dim) and q_plain.is_contiguous() and q_wide.is_contiguous()
    assert q_wide.shape[:2] == (tokens, heads) and at + rot <= q_wide.shape[2] and q_wide.dtype == q_plain.dtype
    assert freq.dtype == torch.float64 and freq.shape[0] >= rot_dims // 2
    lib = library.load()
    check(lib.lse_latent_query(proj.data_ptr(), code, n_partials, stride, ld, q_off, heads, dim, rot, rot_dims,
                               freq.data_ptr(), float(rot_factor), positions.data_ptr(), segment_of_token.data_ptr(),
                               q_plain.data_ptr(), q_wide.data_ptr(), dtype_code(q_plain.dtype), q_wide.shape[2], at,
                               tokens, _stream()), "latent_query")


def latent_attention_mma_supported(dk: int, dv: int, dtype: torch.dtype, window: int = 0) -> bool:
    """Whether the tensor-core kernel takes this shape (bfloat16, DK a multiple of 16, DV a multiple of 8 up to 512,
    no window); other shapes, and float32, run the general kernel."""
    if dtype != torch.bfloat16 or window > 0:
        return False
    return bool(library.load().lse_latent_attention_mma_supported(int(dk), int(dv)))


def latent_attention(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_tables: torch.Tensor,
                     segment_of_token: torch.Tensor, positions: torch.Tensor, scale: float,
                     sink: torch.Tensor | None = None, window: int = 0, split: bool | None = None,
                     segment_start: torch.Tensor | None = None,
                     segment_first_position: torch.Tensor | None = None, tensor_cores: bool = True) -> torch.Tensor:
    """Attention of every row of the step over its request's cached latent rows: q [T, heads, DK], cache
    [pages, page_size, DK], out [T, heads, DV] with DV <= DK: the first DV columns of a row are its value.
    ``sink`` float32 [heads]: exp(sink_h) joins the softmax's denominator.  ``split``: every chunk of 256 keys of a
    row gets a block of its own and a second kernel merges them (default: with few rows).  Given the step's
    ``segment_start`` (int32 [S + 1]) and ``segment_first_position`` (int32 [S]), bfloat16 shapes that the
    tensor-core kernel takes run there (``tensor_cores=False``: the general kernel, for comparisons)."""
    _need_cuda(q, cache, out, block_tables, segment_of_token, positions, sink, segment_start, segment_first_position)
    tokens, heads, dk = q.shape
    dv = out.shape[2]
    page_size = cache.shape[1]
    assert q.is_contiguous() and out.is_contiguous() and cache.is_contiguous() and cache.shape[2] == dk
    assert out.shape[:2] == (tokens, heads) and q.dtype == out.dtype == cache.dtype
    assert block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.stride(1) == 1
    assert sink is None or (sink.dtype == torch.float32 and sink.shape == (heads,))
    lib = library.load()
    partials, max_chunks = None, 0
    if split if split is not None else tokens <= GENERIC_SPLIT_MAX_ROWS:
        chunk = int(lib.lse_latent_attention_chunk())
        max_chunks = max(1, -(-(block_tables.stride(0) * page_size) // chunk))
        partials = torch.empty(tokens * heads * max_chunks * (dv + 2), dtype=torch.float32, device=q.device)
    if (tensor_cores and segment_start is not None and segment_first_position is not None
            and latent_attention_mma_supported(dk, dv, q.dtype, window)):
        segments = segment_first_position.shape[0]
        assert segment_start.dtype == torch.int32 and segment_start.shape[0] == segments + 1
        assert segments == block_tables.shape[0]
        check(lib.lse_latent_attention_mma(q.data_ptr(), cache.data_ptr(), out.data_ptr(), block_tables.data_ptr(),
                                           block_tables.stride(0), segment_start.data_ptr(),
                                           segment_first_position.data_ptr(), _ptr(sink), tokens, segments, heads, dk,
                                           dv, page_size, float(scale), cache.shape[0], _ptr(partials), max_chunks,
                                           _stream()), "latent_attention_mma")
        if partials is not None:
            check(lib.lse_latent_attention_merge(partials.data_ptr(), out.data_ptr(), dtype_code(out.dtype),
                                                 segment_of_token.data_ptr(), positions.data_ptr(), _ptr(sink), tokens,
                                                 heads, dv, 0, max_chunks, block_tables.shape[0], _stream()),
                  "latent_attention_merge")
        return out
    check(lib.lse_latent_attention(q.data_ptr(), cache.data_ptr(), out.data_ptr(), dtype_code(q.dtype),
                                   block_tables.data_ptr(), block_tables.stride(0), segment_of_token.data_ptr(),
                                   positions.data_ptr(), _ptr(sink), tokens, heads, dk, dv, page_size, float(scale),
                                   int(window), cache.shape[0], block_tables.shape[0], _ptr(partials), max_chunks,
                                   _stream()), "latent_attention")
    return out


def head_gemm(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gate: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, h, n] = gate[t, h] * sum_k a[t, h, k] * weight[h, k, n]: a product per head.  a [T, heads, K] and out
    [T, heads, N] may be views with strided rows and heads (innermost contiguous); weight [heads, K, N] any strides
    (pass a transposed view for matrices stored [N, K]); gate float32 [T, heads] or None."""
    _need_cuda(a, weight, out, gate)
    tokens, heads, k = a.shape
    n = out.shape[2]
    assert weight.shape == (heads, k, n) and out.shape[:2] == (tokens, heads)
    assert a.stride(2) == 1 and out.stride(2) == 1
    assert gate is None or (gate.dtype == torch.float32 and gate.shape == (tokens, heads) and gate.is_contiguous())
    lib = library.load()
    check(lib.lse_head_gemm(a.data_ptr(), dtype_code(a.dtype), a.stride(0), a.stride(1), weight.data_ptr(),
                            dtype_code(weight.dtype), weight.stride(0), weight.stride(1), weight.stride(2),
                            out.data_ptr(), dtype_code(out.dtype), out.stride(0), out.stride(1), _ptr(gate), tokens,
                            heads, n, k, _stream()), "head_gemm")
    return out


# ------------------------------------------------------------------ learned positions, norm after the sum, soft cap
def embedding_positions(table: torch.Tensor, pos_table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor,
                        scale: float, residual: torch.Tensor, hidden_out: torch.Tensor | None) -> None:
    """residual[t] = table[ids[t]] * scale + pos_table[positions[t]] in float32; ``hidden_out`` (the tables' dtype, or
    None) receives the same rows rounded."""
    _need_cuda(table, pos_table, ids, positions, residual, hidden_out)
    vocab, hidden = table.shape
    assert pos_table.dtype == table.dtype and pos_table.shape[1] == hidden and table.is_contiguous() and pos_table.is_contiguous()
    assert ids.dtype == torch.int32 and positions.dtype == torch.int32 and residual.dtype == torch.float32
    assert residual.shape == (ids.shape[0], hidden) and residual.is_contiguous()
    assert hidden_out is None or (hidden_out.shape == residual.shape and hidden_out.dtype == table.dtype and hidden_out.is_contiguous())
    check(library.load().lse_embedding_positions(table.data_ptr(), pos_table.data_ptr(), dtype_code(table.dtype),
                                                 ids.data_ptr(), positions.data_ptr(), float(scale), residual.data_ptr(),
                                                 _ptr(hidden_out), ids.shape[0], hidden, vocab, pos_table.shape[0],
                                                 _stream()), "embedding_positions")


def scaled_add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, bias: torch.Tensor | None,
                       row_scale: torch.Tensor | None, alpha: float, weight: torch.Tensor, eps: float,
                       hidden_io: torch.Tensor | None) -> None:
    """residual <- rmsnorm(alpha * residual + delta + bias + row_scale[t] * x_t) * weight, where x_t is the row's value in
    ``hidden_io`` (the residual's copy in the compute dtype, overwritten with the new rows; None: the residual itself
    is the only copy).  delta [T, H], a float32 stack of partial sums [P, T, H], or None; bias float32 [H] or None."""
    _need_cuda(residual, delta, bias, row_scale, weight, hidden_io)
    tokens, hidden = residual.shape
    assert residual.dtype == torch.float32 and residual.is_contiguous() and weight.dtype == torch.float32 and weight.shape == (hidden,)
    assert bias is None or (bias.dtype == torch.float32 and bias.shape == (hidden,))
    assert row_scale is None or (row_scale.dtype == torch.float32 and row_scale.shape[0] >= tokens and row_scale.is_contiguous())
    assert hidden_io is None or (hidden_io.shape == residual.shape and hidden_io.is_contiguous())
    delta, n_partials, stride = _partials(delta, tokens, hidden)
    out_code = dtype_code(hidden_io.dtype) if hidden_io is not None else F32
    delta_code = dtype_code(delta.dtype) if delta is not None else out_code
    check(library.load().lse_scaled_add_rmsnorm(residual.data_ptr(), _ptr(delta), delta_code, n_partials, stride, _ptr(bias),
                                                _ptr(row_scale), float(alpha), weight.data_ptr(), _ptr(hidden_io), out_code,
                                                tokens, hidden, float(eps), _stream()), "scaled_add_rmsnorm")


def softcap(values: torch.Tensor, cap: float) -> torch.Tensor:
    """values <- cap * tanh(values / cap), in place (float32)."""
    _need_cuda(values)
    assert values.dtype == torch.float32 and values.is_contiguous()
    check(library.load().lse_softcap(values.data_ptr(), values.numel(), float(cap), _stream()), "softcap")
    return values


# ------------------------------------------------------------------ attention with normed heads and changed scores
def head_norm_kv_write(proj: torch.Tensor, bias: torch.Tensor | None, q_norm: torch.Tensor | None,
                       k_norm: torch.Tensor | None, eps: float, slot_mapping: torch.Tensor | None, q_out: torch.Tensor,
                       k_cache: torch.Tensor | None, v_cache: torch.Tensor | None, n_q: int, n_kv: int, dk: int,
                       dv: int) -> None:
    """From a row [q (n_q * dk) | k (n_kv * dk) | v (n_kv * dv) | ...] of ``proj`` (+ ``bias``): every query head
    RMS-normed with ``q_norm`` [dk] into ``q_out`` [T, n_q, dk]; every key head normed with ``k_norm`` and every value
    head as it is into the row's place in the pages (k_cache [pages, n_kv, page, dk], v_cache [.., dv]).  ``n_kv`` = 0:
    queries only (a layer that reads another layer's pages)."""
    _need_cuda(proj, bias, q_norm, k_norm, slot_mapping, q_out, k_cache, v_cache)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens = proj.shape[-2]
    assert q_out.shape == (tokens, n_q, dk) and q_out.is_contiguous()
    assert bias is None or bias.dtype == torch.float32
    for weight in (q_norm, k_norm):
        assert weight is None or (weight.dtype == torch.float32 and weight.shape == (dk,))
    page_size = num_pages = 0
    if n_kv:
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == v_cache.dtype == q_out.dtype
        assert k_cache.shape[1] == n_kv and k_cache.shape[3] == dk and v_cache.shape[3] == dv
        assert slot_mapping.dtype == torch.int32 and slot_mapping.shape[0] >= tokens
        num_pages, page_size = k_cache.shape[0], k_cache.shape[2]
    check(library.load().lse_head_norm_kv_write(proj.data_ptr(), code, n_partials, stride, ld, _ptr(bias), _ptr(q_norm),
                                                _ptr(k_norm), float(eps), _ptr(slot_mapping), q_out.data_ptr(),
                                                _ptr(k_cache) if n_kv else None, _ptr(v_cache) if n_kv else None,
                                                dtype_code(q_out.dtype), tokens, n_q, n_kv, dk, dv, page_size, num_pages,
                                                _stream()), "head_norm_kv_write")


def head_norm_rope_kv_write(proj: torch.Tensor, bias: torch.Tensor | None, q_norm: torch.Tensor | None,
                            k_norm: torch.Tensor | None, eps: float, slot_mapping: torch.Tensor, positions: torch.Tensor,
                            freq: torch.Tensor, rot_factor: float, q_out: torch.Tensor, k_cache: torch.Tensor,
                            v_cache: torch.Tensor, n_q: int, n_kv: int, dk: int, dv: int, offset: int = 0) -> None:
    """As :func:`head_norm_kv_write` (the row [q | k | v] starts at column ``offset`` of ``proj``; ``bias`` counts from
    there), and behind the norm the first ``2 * len(freq)`` values of every query and key head
    are rotated: value i with value i + len(freq), by the angle position * freq[i] (``freq`` float64, the angle formed
    in double precision); cosine and sine are multiplied by ``rot_factor``.  Heads up to 256 wide."""
    _need_cuda(proj, bias, q_norm, k_norm, slot_mapping, positions, freq, q_out, k_cache, v_cache)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens = proj.shape[-2]
    assert q_out.shape == (tokens, n_q, dk) and q_out.is_contiguous()
    assert bias is None or bias.dtype == torch.float32
    for weight in (q_norm, k_norm):
        assert weight is None or (weight.dtype == torch.float32 and weight.shape == (dk,))
    assert freq.dtype == torch.float64 and freq.is_contiguous() and positions.dtype == torch.int32
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == v_cache.dtype == q_out.dtype
    assert k_cache.shape[1] == n_kv and k_cache.shape[3] == dk and v_cache.shape[3] == dv
    assert slot_mapping.dtype == torch.int32 and slot_mapping.shape[0] >= tokens
    check(library.load().lse_head_norm_rope_kv_write(
        proj.data_ptr() + int(offset) * proj.element_size(), code, n_partials, stride, ld, _ptr(bias), _ptr(q_norm), _ptr(k_norm), float(eps),
        slot_mapping.data_ptr(), positions.data_ptr(), freq.data_ptr() if freq.numel() else None, float(rot_factor),
        2 * freq.numel(), q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), dtype_code(q_out.dtype), tokens, n_q,
        n_kv, dk, dv, k_cache.shape[2], k_cache.shape[0], _stream()), "head_norm_rope_kv_write")


def attention_scored(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                     block_tables: torch.Tensor, segment_of_token: torch.Tensor, positions: torch.Tensor, scale: float,
                     r1: torch.Tensor | None = None, r2: torch.Tensor | None = None, sink: torch.Tensor | None = None,
                     cross: bool = False, split: bool | None = None, segment_start: torch.Tensor | None = None,
                     segment_first_position: torch.Tensor | None = None, tensor_cores: bool = True,
                     window: int = 0, cap: float = 0.0, head_bias: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of every row of the step over its request's pages, with the scores or weights changed:
    s_ij = q_i . k_j * scale - r1_h ln(1 + r2_h (i - j)) (``r1``, ``r2`` float32 [n_q]); exp(sink_h) in the
    denominator (``sink`` float32 [n_q]).  q [T, n_q, dk]; k_cache [pages, n_kv, page, dk]; v_cache [.., dv];
    out [T, n_q, dv], or with ``cross`` [T, n_q, n_kv, dv]: head h's weights applied to the values of every
    key/value head.  ``out`` is in the cache's dtype or float32.  ``split`` as for :func:`paged_attention_generic`.
    Given the step's ``segment_start`` (int32 [S + 1]) and ``segment_first_position`` (int32 [S]), bfloat16 shapes that
    the tensor-core kernel takes run there (``tensor_cores=False``: the general kernel, for comparisons).
    ``window`` > 0: a row reads its last ``window`` keys only (itself included).  ``cap`` > 0: scores become
    cap * tanh(s / cap).  ``head_bias`` (float32 [n_q]): no softmax; a key's weight is sigmoid(s + head_bias_h) and the
    weights are not normalised over the keys."""
    _need_cuda(q, k_cache, v_cache, out, block_tables, segment_of_token, positions, r1, r2, sink, segment_start,
               segment_first_position, head_bias)
    tokens, n_q, dk = q.shape
    n_kv, page_size, dv = k_cache.shape[1], k_cache.shape[2], v_cache.shape[3]
    n_values = n_kv if cross else 1
    if dk > 256 or dv > 256:
        raise KernelError(f"attention: head sizes {dk}, {dv} beyond 256")
    if n_q % n_kv:
        raise KernelError(f"attention: {n_q} query heads do not divide into {n_kv} groups")
    assert q.is_contiguous() and out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert out.numel() == tokens * n_q * n_values * dv and out.dtype in (q.dtype, torch.float32)
    assert q.dtype == k_cache.dtype == v_cache.dtype and k_cache.shape[3] == dk and v_cache.shape[:3] == k_cache.shape[:3]
    assert block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.stride(1) == 1
    for vector in (r1, r2, sink, head_bias):
        assert vector is None or (vector.dtype == torch.float32 and vector.shape == (n_q,))
    lib = library.load()
    partials, max_chunks = None, 0
    if split if split is not None else tokens <= GENERIC_SPLIT_MAX_ROWS:
        chunk = int(lib.lse_attention_scored_chunk())
        max_chunks = max(1, -(-(block_tables.stride(0) * page_size) // chunk))
        partials = torch.empty(tokens * n_q * n_values * max_chunks * (dv + 2), dtype=torch.float32, device=q.device)
    if (tensor_cores and segment_start is not None and segment_first_position is not None
            and attention_scored_mma_supported(dk, dv, n_q, n_kv, q.dtype)):
        segments = segment_first_position.shape[0]
        assert segment_start.dtype == torch.int32 and segment_start.shape[0] == segments + 1 and segments == block_tables.shape[0]
        check(lib.lse_attention_scored_mma_windowed(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), int(out.dtype == torch.float32),
            block_tables.data_ptr(), block_tables.stride(0), segment_start.data_ptr(), segment_first_position.data_ptr(),
            segments, _ptr(r1), _ptr(r2), _ptr(sink), tokens, n_q, n_kv, dk, dv, int(cross), page_size, float(scale),
            k_cache.shape[0], _ptr(partials), max_chunks, int(window), float(cap), _ptr(head_bias), _stream()),
            "attention_scored_mma")
        if partials is not None:
            check(lib.lse_attention_scored_merge_windowed(
                partials.data_ptr(), out.data_ptr(), dtype_code(out.dtype), segment_of_token.data_ptr(),
                positions.data_ptr(), _ptr(sink), tokens, n_q, n_values, dv, max_chunks, block_tables.shape[0],
                int(window), int(head_bias is not None), _stream()), "attention_scored_merge")
        return out
    check(lib.lse_attention_scored_windowed(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), dtype_code(q.dtype),
        int(out.dtype == torch.float32 and q.dtype != torch.float32), block_tables.data_ptr(), block_tables.stride(0),
        segment_of_token.data_ptr(), positions.data_ptr(), _ptr(r1), _ptr(r2), _ptr(sink), tokens, n_q, n_kv, dk, dv,
        int(cross), page_size, float(scale), k_cache.shape[0], block_tables.shape[0], _ptr(partials), max_chunks,
        int(window), float(cap), _ptr(head_bias), _stream()), "attention_scored")
    return out


def head_mix_gate_stages(n_q: int, n_values: int, dv: int) -> bool:
    """Whether :func:`head_mix_gate` keeps a token's rows in shared memory at this shape (it takes bfloat16 rows only then)."""
    return bool(library.load().lse_head_mix_gate_stages(int(n_q), int(n_values), int(dv)))


def attention_scored_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                        block_tables: torch.Tensor, segment_start: torch.Tensor, segment_first_position: torch.Tensor,
                        scale: float, r1: torch.Tensor | None = None, r2: torch.Tensor | None = None,
                        sink: torch.Tensor | None = None, cross: bool = False) -> torch.Tensor:
    """:func:`attention_scored` for prompt portions on the 5th-generation tensor cores (the kernel of
    :func:`paged_attention_prefill_tc` with the penalty, the sink and the value head as a grid dimension): bfloat16,
    keys and values of one size, 64 or 128, pages of 8 to 128 keys.  out [T, n_q, dv] or, with ``cross``,
    [T, n_q, n_kv, dv], bfloat16.  Every request of the step is worked on in tiles of 128 rows."""
    _need_cuda(q, k_cache, v_cache, out, block_tables, segment_start, segment_first_position, r1, r2, sink)
    tokens, n_q, head_dim = q.shape
    pages, n_kv, page_size = k_cache.shape[0], k_cache.shape[1], k_cache.shape[2]
    segments = segment_first_position.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert v_cache.shape == k_cache.shape and k_cache.shape[3] == head_dim
    assert out.numel() == tokens * n_q * (n_kv if cross else 1) * head_dim
    assert block_tables.dtype == torch.int32 and block_tables.stride(1) == 1 and segment_start.shape[0] == segments + 1
    for vector in (r1, r2, sink):
        assert vector is None or (vector.dtype == torch.float32 and vector.shape == (n_q,))
    scratch, counters = _attention_tc_scratch(q.device)
    check(library.load().lse_attention_scored_tc(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                                 block_tables.data_ptr(), block_tables.stride(0), segment_start.data_ptr(),
                                                 segment_first_position.data_ptr(), segments, tokens, pages, n_q, n_kv,
                                                 head_dim, page_size, float(scale), _ptr(r1), _ptr(r2), _ptr(sink),
                                                 int(cross), _ptr(scratch), _ptr(counters), counters.shape[0], _stream()),
          "attention_scored_tc")
    return out


def attention_sigmoid_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                         block_tables: torch.Tensor, segment_start: torch.Tensor, segment_first_position: torch.Tensor,
                         scale: float, head_bias: torch.Tensor, cap: float = 0.0) -> torch.Tensor:
    """:func:`attention_scored` with ``head_bias`` (weights sigmoid(capped score + head_bias_h), not normalised over the
    keys) for prompt portions on the 5th-generation tensor cores: the shapes of :func:`attention_scored_tc`; out
    [T, n_q, dv] bfloat16.  Every request of the step is worked on in tiles of 128 rows."""
    _need_cuda(q, k_cache, v_cache, out, block_tables, segment_start, segment_first_position, head_bias)
    tokens, n_q, head_dim = q.shape
    pages, n_kv, page_size = k_cache.shape[0], k_cache.shape[1], k_cache.shape[2]
    segments = segment_first_position.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert v_cache.shape == k_cache.shape and k_cache.shape[3] == head_dim and out.numel() == tokens * n_q * head_dim
    assert block_tables.dtype == torch.int32 and block_tables.stride(1) == 1 and segment_start.shape[0] == segments + 1
    assert head_bias.dtype == torch.float32 and head_bias.shape == (n_q,)
    scratch, counters = _attention_tc_scratch(q.device)
    check(library.load().lse_attention_sigmoid_tc(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                                  block_tables.data_ptr(), block_tables.stride(0), segment_start.data_ptr(),
                                                  segment_first_position.data_ptr(), segments, tokens, pages, n_q, n_kv,
                                                  head_dim, page_size, float(scale), head_bias.data_ptr(), float(cap),
                                                  _ptr(scratch), _ptr(counters), counters.shape[0], _stream()),
          "attention_sigmoid_tc")
    return out


def attention_scored_mma_supported(dk: int, dv: int, n_q: int, n_kv: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core form of :func:`attention_scored` takes this shape (bfloat16; keys and values of one
    size, 32, 48, 64, 96 or 128; at most 64 query heads a group)."""
    if dtype != torch.bfloat16:
        return False
    return bool(library.load().lse_attention_scored_mma_supported(int(dk), int(dv), int(n_q), int(n_kv)))


def head_mix_gate(wide: torch.Tensor, mix: torch.Tensor | None, gate_proj: torch.Tensor | None, gate_offset: int,
                  gate_bias: torch.Tensor | None, segment_of_token: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int,
                  dv: int) -> torch.Tensor:
    """out[t, h] = sigmoid(gate)[t, h] * sum_g mix[h, g] * wide[t, g, slot of h]: ``wide`` [T, n_q, n_kv, dv] in float32
    or bfloat16 (the output of :func:`attention_scored` with ``cross``; the slot of h is its own key/value head) or [T, n_q, dv];
    ``mix`` float32 [n_q, n_q] or None; the gate's pre-activation is columns ``gate_offset`` .. + n_q * dv of
    ``gate_proj`` (+ ``gate_bias`` float32 [n_q * dv]), or None for no gate; out [T, n_q * dv]."""
    _need_cuda(wide, mix, gate_proj, gate_bias, segment_of_token, out)
    tokens = out.shape[0]
    cross = wide.numel() == tokens * n_q * n_kv * dv and n_kv > 1
    assert wide.dtype in (torch.float32, torch.bfloat16) and wide.is_contiguous()
    assert wide.numel() == tokens * n_q * (n_kv if cross else 1) * dv
    assert out.shape == (tokens, n_q * dv) and out.is_contiguous()
    assert mix is None or (mix.dtype == torch.float32 and mix.shape == (n_q, n_q) and mix.is_contiguous())
    code, n_partials, stride, ld, pointer = dtype_code(out.dtype), 1, 0, 0, None
    if gate_proj is not None:
        gate_proj, code, n_partials, stride, ld = _projection(gate_proj)
        pointer = gate_proj.data_ptr() + gate_offset * gate_proj.element_size()
        assert gate_bias is None or (gate_bias.dtype == torch.float32 and gate_bias.shape == (n_q * dv,))
    check(library.load().lse_head_mix_gate(wide.data_ptr(), int(wide.dtype == torch.bfloat16), _ptr(mix), pointer, code, n_partials, stride, ld,
                                           _ptr(gate_bias) if gate_proj is not None else None, segment_of_token.data_ptr(),
                                           out.data_ptr(), dtype_code(out.dtype), tokens, n_q, n_kv, int(cross), dv,
                                           _stream()), "head_mix_gate")
    return out


# ------------------------------------------------------------------ mixture of experts
def moe_route(logits: torch.Tensor, correction: torch.Tensor | None, outputs: int, identity: int, top: int,
              shared_gate: bool = False, chosen: torch.Tensor | None = None, logit_bias: torch.Tensor | None = None,
              over_chosen: bool = False):
    """The router of a mixture of experts, in float32.  ``logits`` float32 [T, N] (or a stack of partial sums [P, T, N]):
    column e < ``outputs`` is router output e (the last ``identity`` of them identity experts), column ``outputs`` the
    pre-activation of the shared expert's gate when ``shared_gate``; further columns are padding.  Scores softmax(z)
    over the outputs, the ``top`` largest of score + ``correction`` chosen, weights the scores themselves.  Returns
    (expert_weights float32 [T, experts], zero where not chosen; identity_weight float32 [T], the chosen identity
    experts' weights added up; the shared gate float32 [T] = sigmoid of its column, or None).  ``chosen`` int32
    [T, top] receives the choices.  ``logit_bias`` (float32 [outputs]) is added to the logits.  ``over_chosen``: the
    largest logits are chosen and the weights are the softmax over the chosen logits only."""
    _need_cuda(logits, correction, chosen, logit_bias)
    assert logit_bias is None or (logit_bias.dtype == torch.float32 and logit_bias.shape == (outputs,))
    logits, code, n_partials, stride, ld = _projection(logits)
    tokens = logits.shape[-2]
    assert code == F32 and logits.shape[-1] >= outputs + int(shared_gate)
    assert correction is None or (correction.dtype == torch.float32 and correction.shape == (outputs,))
    assert chosen is None or (chosen.dtype == torch.int32 and chosen.shape == (tokens, top) and chosen.is_contiguous())
    expert_weights = torch.empty((tokens, outputs - identity), dtype=torch.float32, device=logits.device)
    identity_weight = torch.empty((tokens,), dtype=torch.float32, device=logits.device)
    gate = torch.empty((tokens,), dtype=torch.float32, device=logits.device) if shared_gate else None
    check(library.load().lse_moe_route_biased(logits.data_ptr(), n_partials, stride, ld, _ptr(correction),
                                              int(shared_gate), expert_weights.data_ptr(), identity_weight.data_ptr(),
                                              _ptr(gate), _ptr(chosen), tokens, int(outputs), int(identity), int(top),
                                              _ptr(logit_bias), int(over_chosen), _stream()), "moe_route")
    return expert_weights, identity_weight, gate


def moe_route_sigmoid(logits: torch.Tensor, correction: torch.Tensor | None, experts: int, top: int, group_count: int,
                      group_keep: int, scale: float, shared_gate: bool = False, chosen: torch.Tensor | None = None):
    """A router with sigmoid scores, in float32: s = sigmoid(z); the choice goes by s + ``correction`` and is confined to
    the ``group_keep`` best of ``group_count`` equal groups of neighbouring experts (a group's score: the sum of its two
    largest choice scores); the ``top`` largest choice scores are chosen; weights s / (sum of the chosen s + 1e-20) *
    ``scale``.  ``group_count`` <= 1: no groups.  Arguments and results otherwise as :func:`moe_route` (no identity
    experts: the second result is zeros)."""
    _need_cuda(logits, correction, chosen)
    logits, code, n_partials, stride, ld = _projection(logits)
    tokens = logits.shape[-2]
    assert code == F32 and logits.shape[-1] >= experts + int(shared_gate)
    assert correction is None or (correction.dtype == torch.float32 and correction.shape == (experts,))
    assert chosen is None or (chosen.dtype == torch.int32 and chosen.shape == (tokens, top) and chosen.is_contiguous())
    expert_weights = torch.empty((tokens, experts), dtype=torch.float32, device=logits.device)
    identity_weight = torch.empty((tokens,), dtype=torch.float32, device=logits.device)
    gate = torch.empty((tokens,), dtype=torch.float32, device=logits.device) if shared_gate else None
    check(library.load().lse_moe_route_sigmoid(logits.data_ptr(), n_partials, stride, ld, _ptr(correction),
                                               int(shared_gate), expert_weights.data_ptr(), identity_weight.data_ptr(),
                                               _ptr(gate), _ptr(chosen), tokens, int(experts), int(top), int(group_count),
                                               int(group_keep), float(scale), _stream()), "moe_route_sigmoid")
    return expert_weights, identity_weight, gate


MOE_ACTIVATIONS = {"clamped_swish": 0, "silu": 1, "squared_relu": 2}
MOE_UNGATED = frozenset({"squared_relu"})    # activations of experts without a gate: one input column per output column


def moe_gated_act(gate_up: torch.Tensor, expert_weights: torch.Tensor, shared_gate: torch.Tensor | None,
                  out: torch.Tensor, experts: int, ff: int, shared_ff: int, limit: float, shared_limit: float,
                  valid_rows: torch.Tensor | None = None, activation: str = "clamped_swish") -> torch.Tensor:
    """out[t, i] = c * g * sigmoid(1.702 g) * (u + 1) with g = min(gate_i, limit), u = clamp(up_i, -limit, limit), over
    the columns of all experts side by side (``experts`` blocks of ``ff``, then ``shared_ff`` of the shared expert with
    its own limit); c is the token's weight of the column's expert (``shared_gate`` for the shared columns; 1 where
    the weights are None).  ``gate_up`` is [T, 2 I] (expert by expert [gate | up], then the shared expert's
    [gate | up]) or a float32 stack of partial sums.  ``valid_rows`` (int32, one number on the device): rows from it on
    may be left alone (the unused end of a buffer grouped by expert).  ``activation`` "silu": out = c * silu(g) * u with
    nothing clamped; "squared_relu": experts without a gate, ``gate_up`` is [T, I] (one column per output column) and
    out = c * relu(u)^2."""
    _need_cuda(gate_up, expert_weights, shared_gate, out, valid_rows)
    tokens, inter = out.shape
    columns = inter if activation in MOE_UNGATED else 2 * inter
    assert inter == experts * ff + shared_ff and out.is_contiguous() and gate_up.shape[-1] == columns
    gate_up, n_partials, stride = _partials(gate_up, tokens, columns)
    assert expert_weights is None or (expert_weights.dtype == torch.float32 and expert_weights.shape == (tokens, experts)
                                      and expert_weights.is_contiguous())
    check(library.load().lse_moe_gated_act_kind(gate_up.data_ptr(), dtype_code(gate_up.dtype), n_partials, stride,
                                                _ptr(expert_weights), _ptr(shared_gate), out.data_ptr(),
                                                dtype_code(out.dtype), tokens, experts, ff, shared_ff, float(limit),
                                                float(shared_limit), _ptr(valid_rows),
                                                MOE_ACTIVATIONS[activation], _stream()), "moe_gated_act")
    return out


def moe_group_rows(chosen: torch.Tensor, experts: int, segment_of_token: torch.Tensor | None = None):
    """Places for the rows of a grouped product: ``chosen`` int32 [T, top] (a router's choices; ids from ``experts`` on
    are identity experts and get no row).  Returns (row_of int32 [T, top]: the row of every (token, choice), -1 for
    none; offsets int32 [experts]: the end of every expert's range of rows).  Rows of padding tokens
    (``segment_of_token`` < 0) get no place."""
    _need_cuda(chosen, segment_of_token)
    tokens, top = chosen.shape
    assert chosen.dtype == torch.int32 and chosen.is_contiguous()
    row_of = torch.empty_like(chosen)
    offsets = torch.empty((experts,), dtype=torch.int32, device=chosen.device)
    check(library.load().lse_moe_group_rows(chosen.data_ptr(), _ptr(segment_of_token), row_of.data_ptr(), offsets.data_ptr(),
                                            tokens, top, int(experts), _stream()), "moe_group_rows")
    return row_of, offsets


def moe_gather_rows(x: torch.Tensor, row_of: torch.Tensor, grouped: torch.Tensor) -> torch.Tensor:
    """grouped[row_of[t, k]] = x[t] for every place that is not -1."""
    _need_cuda(x, row_of, grouped)
    tokens, top = row_of.shape
    assert x.is_contiguous() and grouped.is_contiguous() and x.dtype == grouped.dtype and x.shape[1] == grouped.shape[1]
    assert grouped.shape[0] >= tokens * top and x.shape[0] == tokens
    check(library.load().lse_moe_gather_rows(x.data_ptr(), dtype_code(x.dtype), row_of.data_ptr(), grouped.data_ptr(),
                                             tokens, top, x.shape[1], _stream()), "moe_gather_rows")
    return grouped


def moe_combine(down: torch.Tensor, row_of: torch.Tensor, chosen: torch.Tensor, expert_weights: torch.Tensor,
                identity_weight: torch.Tensor | None, x: torch.Tensor, y: torch.Tensor, accumulate: bool) -> torch.Tensor:
    """y[t] (+)= sum_k expert_weights[t, chosen[t, k]] * down[row_of[t, k]] + identity_weight[t] * x[t], the sum in the
    order of the token's choices; y float32 [T, W] (``accumulate``: it holds something already, else it is overwritten)."""
    _need_cuda(down, row_of, chosen, expert_weights, identity_weight, x, y)
    tokens, top = row_of.shape
    assert y.dtype == torch.float32 and y.is_contiguous() and y.shape == x.shape and x.is_contiguous() and down.is_contiguous()
    assert down.dtype == x.dtype and down.shape[1] == x.shape[1] and expert_weights.is_contiguous()
    check(library.load().lse_moe_combine(down.data_ptr(), dtype_code(down.dtype), row_of.data_ptr(), chosen.data_ptr(),
                                         expert_weights.data_ptr(), _ptr(identity_weight), x.data_ptr(), y.data_ptr(),
                                         tokens, x.shape[1], top, expert_weights.shape[1], int(accumulate), _stream()),
          "moe_combine")
    return y


# ------------------------------------------------------------------ the tanh norm
def tanh_norm(residual: torch.Tensor, delta: torch.Tensor | None, after, before, out: torch.Tensor | None,
              rows: torch.Tensor | None = None, write_residual: bool = True) -> torch.Tensor | None:
    """residual += after(delta); out = before(residual[rows]), with the tanh norm f(x) = tanh(alpha x) * w + b.
    ``after`` and ``before`` are (alpha float32 [1], w float32 [H], b float32 [H]) or None (``after`` None: the output is
    added as it is; ``before`` None with ``out`` None: only the sum).  residual float32 [T, H]; delta [T, H] or a float32
    stack of partial sums; out [R, H] in float32 or bfloat16, R = len(rows) or T."""
    _need_cuda(residual, delta, out, rows)
    tokens, hidden = residual.shape
    assert residual.dtype == torch.float32 and residual.is_contiguous()
    delta, n_partials, stride = _partials(delta, tokens, hidden)
    for triple in (after, before):
        if triple is not None:
            alpha, weight, bias = triple
            assert alpha.dtype == weight.dtype == bias.dtype == torch.float32 and alpha.numel() == 1
            assert weight.shape == (hidden,) and bias.shape == (hidden,)
    n_rows = tokens if rows is None else rows.shape[0]
    if out is not None:
        assert before is not None and out.shape == (n_rows, hidden) and out.is_contiguous()
    assert rows is None or rows.dtype == torch.int32
    code = dtype_code(delta.dtype) if delta is not None else F32
    a, b = after or (None, None, None), before or (None, None, None)
    check(library.load().lse_tanh_norm(residual.data_ptr(), _ptr(delta), code, n_partials, stride, _ptr(a[0]), _ptr(a[1]),
                                       _ptr(a[2]), _ptr(b[0]), _ptr(b[1]), _ptr(b[2]), _ptr(out),
                                       dtype_code(out.dtype) if out is not None else F32, _ptr(rows), n_rows, hidden,
                                       int(write_residual), _stream()), "tanh_norm")
    return out


# ------------------------------------------------------------------ matrix memory with exponential gates
def mlstm_gates(proj: torch.Tensor, i_off: int, f_off: int, i_bias: torch.Tensor, f_bias: torch.Tensor, cap: float,
                state_m: torch.Tensor, segment_start: torch.Tensor, segment_slot: torch.Tensor, heads: int):
    """From the gates' pre-activations (columns i_off + h and f_off + h of ``proj``, + bias): i = cap tanh(z / cap),
    f = logsigmoid(cap tanh(z / cap)), m_t = max(f_t + m_(t-1), i_t) along every request's rows from and into
    ``state_m`` float32 [slots, heads].  Returns (keep, take, floor) float32 [T, heads]: exp(f_t + m_(t-1) - m_t),
    exp(i_t - m_t), exp(-m_t)."""
    _need_cuda(proj, i_bias, f_bias, state_m, segment_start, segment_slot)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens = proj.shape[-2]
    assert state_m.dtype == torch.float32 and state_m.is_contiguous() and state_m.shape[1:] == (heads,)
    assert i_bias.dtype == f_bias.dtype == torch.float32 and i_bias.shape == f_bias.shape == (heads,)
    segments = segment_slot.shape[0]
    assert segment_start.dtype == segment_slot.dtype == torch.int32 and segment_start.shape[0] == segments + 1
    keep, take, floor = (torch.empty((tokens, heads), dtype=torch.float32, device=proj.device) for _ in range(3))
    check(library.load().lse_mlstm_gates(proj.data_ptr(), code, n_partials, stride, ld, int(i_off), int(f_off),
                                         i_bias.data_ptr(), f_bias.data_ptr(), float(cap), state_m.data_ptr(),
                                         segment_start.data_ptr(), segment_slot.data_ptr(), keep.data_ptr(),
                                         take.data_ptr(), floor.data_ptr(), segments, heads, state_m.shape[0],
                                         _stream()), "mlstm_gates")
    return keep, take, floor


def gated_linear_attention_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, keep: torch.Tensor,
                                take: torch.Tensor, q_scale: float, state: torch.Tensor, segment_start: torch.Tensor,
                                segment_slot: torch.Tensor, out: torch.Tensor, heads: int, dim: int, vdim: int,
                                chunked: bool | None = None) -> torch.Tensor:
    """S_t = keep[t, h] S_(t-1) + take[t, h] k_t [v_t | 1]^T, out_t = S_t^T (q_scale q_t), over the rows of every request
    in order, from and into ``state`` float32 [slots, heads, dim, vdim + 1] (the last column is the normaliser n, so
    out's last column is n_t . q_t); out float32 [T, heads * (vdim + 1)].  ``chunked`` as for
    :func:`linear_attention_scan`."""
    _need_cuda(proj, keep, take, state, segment_start, segment_slot, out)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens = proj.shape[-2]
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (heads, dim, vdim + 1)
    assert keep.dtype == take.dtype == torch.float32 and keep.shape == take.shape == (tokens, heads)
    assert keep.is_contiguous() and take.is_contiguous()
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == (tokens, heads * (vdim + 1))
    segments = segment_slot.shape[0]
    assert segment_start.dtype == segment_slot.dtype == torch.int32 and segment_start.shape[0] == segments + 1
    chunk_rows, chunk_state, max_chunks = 0, None, 0
    if chunked if chunked is not None else tokens >= LINEAR_ATTENTION_CHUNKED_FROM:
        chunk_rows = LINEAR_ATTENTION_CHUNK
        max_chunks = tokens // chunk_rows + segments
        chunk_state = torch.empty((max_chunks, heads, dim, vdim + 1), dtype=torch.float32, device=out.device)
    check(library.load().lse_gated_linear_attention_scan(
        proj.data_ptr(), code, n_partials, stride, ld, int(q_off), int(k_off), int(v_off), keep.data_ptr(),
        take.data_ptr(), float(q_scale), state.data_ptr(), segment_start.data_ptr(), segment_slot.data_ptr(),
        out.data_ptr(), segments, heads, dim, vdim, state.shape[0], chunk_rows, _ptr(chunk_state), max_chunks, _stream()),
        "gated_linear_attention_scan")
    return out


def ssd_gates(proj: torch.Tensor, dt_off: int, dt_bias: torch.Tensor, a_log: torch.Tensor):
    """(keep, take) float32 [T, heads] of a state-space scan with one decay per head: dt = softplus(proj[:, dt_off + h] +
    dt_bias[h]) (no clamp), keep = exp(-exp(a_log[h]) dt), take = dt."""
    _need_cuda(proj, dt_bias, a_log)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens, heads = proj.shape[-2], dt_bias.shape[0]
    assert dt_bias.dtype == a_log.dtype == torch.float32 and a_log.shape == (heads,)
    keep = torch.empty((tokens, heads), dtype=torch.float32, device=proj.device)
    take = torch.empty_like(keep)
    check(library.load().lse_ssd_gates(proj.data_ptr(), code, n_partials, stride, ld, int(dt_off), dt_bias.data_ptr(),
                                       a_log.data_ptr(), keep.data_ptr(), take.data_ptr(), tokens, heads, _stream()),
          "ssd_gates")
    return keep, take


def sigmoid_power(proj: torch.Tensor, off: int, n: int, bias: torch.Tensor | None, tau: float) -> torch.Tensor:
    """float32 [T, n]: sigmoid(proj[:, off .. off + n] + bias)^(1 / tau), through the logarithm of the sigmoid."""
    _need_cuda(proj, bias)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens = proj.shape[-2]
    assert bias is None or (bias.dtype == torch.float32 and bias.shape == (n,))
    keep = torch.empty((tokens, n), dtype=torch.float32, device=proj.device)
    check(library.load().lse_sigmoid_power(proj.data_ptr(), code, n_partials, stride, ld, int(off), _ptr(bias), float(tau),
                                           keep.data_ptr(), tokens, int(n), _stream()), "sigmoid_power")
    return keep


def _scan_chunks(tokens: int, segments: int, chunked: bool | None):
    if chunked if chunked is not None else tokens >= LINEAR_ATTENTION_CHUNKED_FROM:
        return LINEAR_ATTENTION_CHUNK, tokens // LINEAR_ATTENTION_CHUNK + segments
    return 0, 0


def token_decay_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, keep: torch.Tensor, take: torch.Tensor,
                     q_scale: float, state: torch.Tensor, segment_start: torch.Tensor, segment_slot: torch.Tensor,
                     out: torch.Tensor, heads: int, dim: int, vdim: int, qk_share: int = 1,
                     chunked: bool | None = None) -> torch.Tensor:
    """S_t = keep[t, h] S_(t-1) + take[t, h] k_t v_t^T, out_t = S_t^T (q_scale q_t), as
    :func:`gated_linear_attention_scan` without the normaliser's column (state float32 [slots, heads, dim, vdim], out
    float32 [T, heads * vdim]) and with ``qk_share`` neighbouring heads reading the same q and k columns (head h reads q at
    q_off + (h // qk_share) * dim): a state-space scan whose inputs B (k) and C (q) belong to groups of heads."""
    _need_cuda(proj, keep, take, state, segment_start, segment_slot, out)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens = proj.shape[-2]
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (heads, dim, vdim)
    assert keep.dtype == take.dtype == torch.float32 and keep.shape == take.shape == (tokens, heads)
    assert keep.is_contiguous() and take.is_contiguous() and heads % qk_share == 0
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == (tokens, heads * vdim)
    segments = segment_slot.shape[0]
    assert segment_start.dtype == segment_slot.dtype == torch.int32 and segment_start.shape[0] == segments + 1
    chunk_rows, max_chunks = _scan_chunks(tokens, segments, chunked)
    chunk_state = (torch.empty((max_chunks, heads, dim, vdim), dtype=torch.float32, device=out.device)
                   if chunk_rows else None)
    check(library.load().lse_gated_linear_attention_scan_shared(
        proj.data_ptr(), code, n_partials, stride, ld, int(q_off), int(k_off), int(v_off), keep.data_ptr(),
        take.data_ptr(), float(q_scale), state.data_ptr(), segment_start.data_ptr(), segment_slot.data_ptr(),
        out.data_ptr(), segments, heads, dim, vdim, state.shape[0], chunk_rows, _ptr(chunk_state), max_chunks, 0,
        int(qk_share), _stream()), "token_decay_scan")
    return out


def channel_decay_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, keep: torch.Tensor, q_scale: float,
                       state: torch.Tensor, segment_start: torch.Tensor, segment_slot: torch.Tensor, out: torch.Tensor,
                       heads: int, dim: int, vdim: int, chunked: bool | None = None) -> torch.Tensor:
    """S_t = diag(keep[t, h, :]) S_(t-1) + k_t v_t^T, out_t = S_t^T (q_scale q_t): a decay per row of the state (per key
    channel), token and head; keep float32 [T, heads * dim]; state float32 [slots, heads, dim, vdim]; out float32
    [T, heads * vdim].  ``chunked`` as for :func:`linear_attention_scan`."""
    _need_cuda(proj, keep, state, segment_start, segment_slot, out)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens = proj.shape[-2]
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (heads, dim, vdim)
    assert keep.dtype == torch.float32 and keep.shape == (tokens, heads * dim) and keep.is_contiguous()
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == (tokens, heads * vdim)
    segments = segment_slot.shape[0]
    assert segment_start.dtype == segment_slot.dtype == torch.int32 and segment_start.shape[0] == segments + 1
    chunk_rows, max_chunks = _scan_chunks(tokens, segments, chunked)
    chunk_state = chunk_keep = None
    if chunk_rows:
        chunk_state = torch.empty((max_chunks, heads, dim, vdim), dtype=torch.float32, device=out.device)
        chunk_keep = torch.empty((max_chunks, heads, dim), dtype=torch.float32, device=out.device)
    check(library.load().lse_vector_decay_attention_scan(
        proj.data_ptr(), code, n_partials, stride, ld, int(q_off), int(k_off), int(v_off), keep.data_ptr(), float(q_scale),
        state.data_ptr(), segment_start.data_ptr(), segment_slot.data_ptr(), out.data_ptr(), segments, heads, dim, vdim,
        state.shape[0], chunk_rows, _ptr(chunk_state), max_chunks, _ptr(chunk_keep), _stream()), "channel_decay_scan")
    return out


def gated_group_rmsnorm(values: torch.Tensor, proj: torch.Tensor, g_off: int, weight: torch.Tensor, eps: float,
                        out: torch.Tensor, groups: int, gate_first: bool, gate_activation: str = "silu",
                        scale: float = 1.0, skip: torch.Tensor | None = None, skip_source: torch.Tensor | None = None,
                        skip_offset: int = 0, segment_of_token: torch.Tensor | None = None) -> torch.Tensor:
    """The norm behind a scan, in ``groups`` equal parts of a row, each by its own root mean square.  With a = values
    (+ skip[head] * x, x the columns ``skip_offset`` .. of ``skip_source``, a head being n / len(skip) columns) and g
    the columns ``g_off`` .. of ``proj`` through ``gate_activation`` ("silu" or "sigmoid"):
    ``gate_first``: b = a g, out = b / rms(b) * weight * scale; else out = a / rms(a) * weight * g * scale.
    ``weight`` float32 of any length that divides n, read at column % length (a weight per part shared by the parts).
    ``out`` [T, n] in the compute dtype; its rows may be strided (a column range of a wider tensor)."""
    _need_cuda(values, proj, weight, out, skip, skip_source, segment_of_token)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens, n = values.shape
    assert values.dtype == torch.float32 and values.is_contiguous() and weight.dtype == torch.float32
    assert n % groups == 0 and n % weight.shape[0] == 0 and out.shape == (tokens, n) and out.stride(1) == 1
    x_ld = head_width = 0
    if skip is not None:
        assert skip.dtype == torch.float32 and n % skip.shape[0] == 0 and skip_source.dtype == out.dtype
        assert skip_source.dim() == 2 and skip_source.stride(1) == 1
        x_ld, head_width = skip_source.stride(0), n // skip.shape[0]
    check(library.load().lse_gated_group_rmsnorm(
        values.data_ptr(), proj.data_ptr(), code, n_partials, stride, ld, int(g_off), _ptr(skip_source), x_ld,
        int(skip_offset), _ptr(skip), head_width, weight.data_ptr(), weight.shape[0], out.data_ptr(), dtype_code(out.dtype),
        out.stride(0), tokens, n, int(groups), float(eps), float(scale), int(gate_first),
        {"sigmoid": 0, "silu": 1}[gate_activation], _ptr(segment_of_token), _stream()), "gated_group_rmsnorm")
    return out


def mlstm_readout(read: torch.Tensor, floor: torch.Tensor, proj: torch.Tensor, g_off: int, weight: torch.Tensor,
                  eps: float, out: torch.Tensor, heads: int, vdim: int,
                  segment_of_token: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, h, :] = rms(read[t, h, :vdim] / (max(|read[t, h, vdim]|, floor[t, h]) + 1e-6)) * weight * sigmoid(gate), the
    root mean square taken per head; the gate's pre-activation is columns g_off .. of ``proj``."""
    _need_cuda(read, floor, proj, weight, out, segment_of_token)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens = out.shape[0]
    assert read.dtype == floor.dtype == weight.dtype == torch.float32 and read.is_contiguous() and floor.is_contiguous()
    assert read.shape == (tokens, heads * (vdim + 1)) and floor.shape == (tokens, heads) and weight.shape == (heads * vdim,)
    assert out.shape == (tokens, heads * vdim) and out.is_contiguous()
    check(library.load().lse_mlstm_readout(read.data_ptr(), floor.data_ptr(), proj.data_ptr(), code, n_partials, stride, ld,
                                           int(g_off), weight.data_ptr(), out.data_ptr(), dtype_code(out.dtype), tokens,
                                           heads, vdim, float(eps), _ptr(segment_of_token), _stream()), "mlstm_readout")
    return out


# ------------------------------------------------------------------ short convolutions and what follows them
def short_conv_act(proj: torch.Tensor, off: int, weight: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor,
                   step, out: torch.Tensor, activation: str = "none") -> torch.Tensor:
    """out[t, c] = act(sum_j weight[c, j] u_(t - taps + 1 + j)[c] + bias[c]) where u are columns off .. off + C of
    ``proj`` along the request's rows and, before this step's rows, the request's window in ``state`` float32
    [slots, taps - 1, C].  weight float32 [C, taps]; ``step``: the step's context; ``activation`` "none" or "silu"."""
    _need_cuda(proj, weight, bias, state, out)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens, channels = out.shape
    taps = weight.shape[1]
    assert weight.dtype == torch.float32 and weight.shape == (channels, taps) and weight.is_contiguous()
    assert bias is None or (bias.dtype == torch.float32 and bias.shape == (channels,))
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (taps - 1, channels)
    assert out.is_contiguous() and proj.shape[-2] == tokens
    check(library.load().lse_short_conv_act(proj.data_ptr(), code, n_partials, stride, ld, int(off), weight.data_ptr(),
                                            _ptr(bias), state.data_ptr(), step.segment_of_token.data_ptr(),
                                            step.segment_start.data_ptr(), step.segment_state_slot.data_ptr(),
                                            out.data_ptr(), dtype_code(out.dtype), tokens, channels, taps,
                                            {"none": 0, "silu": 1}[activation], state.shape[0],
                                            step.segment_state_slot.shape[0], _stream()), "short_conv_act")
    return out


def short_conv_state(proj: torch.Tensor, off: int, channels: int, taps: int, state: torch.Tensor, step) -> None:
    """Move every request's window in ``state`` (float32 [slots, taps - 1, channels]) on by the step's rows: afterwards it
    holds the request's last taps - 1 inputs.  Launch it after the kernels that read the old window."""
    _need_cuda(proj, state)
    proj, code, n_partials, stride, ld = _projection(proj)
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (taps - 1, channels)
    check(library.load().lse_short_conv_state(proj.data_ptr(), code, n_partials, stride, ld, int(off), state.data_ptr(),
                                              step.segment_start.data_ptr(), step.segment_state_slot.data_ptr(),
                                              step.segment_state_slot.shape[0], channels, taps, state.shape[0], _stream()),
          "short_conv_state")


def conv_qk_norm_rope(proj: torch.Tensor, off: int, g_off: int, weight: torch.Tensor, state: torch.Tensor,
                      q_norm: torch.Tensor, k_norm: torch.Tensor, eps: float, freq: torch.Tensor, rot_factor: float,
                      step, slot_mapping: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      gate_out: torch.Tensor | None, n_q: int, n_kv: int, dk: int, dv: int) -> None:
    """Columns off .. of ``proj`` are [q (n_q dk) | k (n_kv dk) | v (n_kv dv)]; each passes its short convolution
    (``weight`` float32 [channels, taps], windows in ``state``); q and k are RMS-normed over their whole width
    (``q_norm`` [n_q dk], ``k_norm`` [n_kv dk]) and the first 2 len(freq) values of every head rotated (value i with
    i + len(freq); angle position * freq[i], freq float64; cosine and sine times ``rot_factor``); q goes to ``q_out``
    [T, n_q, dk], k and v into the row's place in the pages.  ``gate_out`` float32 [T, n_q] receives the sigmoid of
    columns g_off .. g_off + n_q."""
    _need_cuda(proj, weight, state, q_norm, k_norm, freq, slot_mapping, q_out, k_cache, v_cache, gate_out)
    proj, code, n_partials, stride, ld = _projection(proj)
    tokens = q_out.shape[0]
    channels, taps = (n_q + n_kv) * dk + n_kv * dv, weight.shape[1]
    assert weight.dtype == torch.float32 and weight.shape == (channels, taps) and weight.is_contiguous()
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (taps - 1, channels)
    assert q_norm.dtype == k_norm.dtype == torch.float32 and q_norm.shape == (n_q * dk,) and k_norm.shape == (n_kv * dk,)
    assert freq.dtype == torch.float64 and freq.is_contiguous() and 2 * freq.shape[0] <= dk
    assert q_out.shape == (tokens, n_q, dk) and q_out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.dtype == v_cache.dtype == q_out.dtype and k_cache.shape[1] == n_kv and k_cache.shape[3] == dk
    assert v_cache.shape[3] == dv and v_cache.shape[:3] == k_cache.shape[:3]
    assert gate_out is None or (gate_out.dtype == torch.float32 and gate_out.shape == (tokens, n_q) and gate_out.is_contiguous())
    assert slot_mapping.dtype == torch.int32 and slot_mapping.shape[0] >= tokens
    check(library.load().lse_conv_qk_norm_rope(
        proj.data_ptr(), code, n_partials, stride, ld, int(off), int(g_off), weight.data_ptr(), state.data_ptr(),
        q_norm.data_ptr(), k_norm.data_ptr(), float(eps), freq.data_ptr(), float(rot_factor), 2 * freq.shape[0],
        step.positions.data_ptr(), step.segment_of_token.data_ptr(), step.segment_start.data_ptr(),
        step.segment_state_slot.data_ptr(), slot_mapping.data_ptr(), q_out.data_ptr(), k_cache.data_ptr(),
        v_cache.data_ptr(), dtype_code(q_out.dtype), _ptr(gate_out), tokens, n_q, n_kv, dk, dv, taps, k_cache.shape[2],
        k_cache.shape[0], state.shape[0], step.segment_state_slot.shape[0], _stream()), "conv_qk_norm_rope")


def head_gate_scale(attended: torch.Tensor, gate: torch.Tensor | None, out: torch.Tensor, scale: float,
                    segment_of_token: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, h * dv + j] = attended[t, h, j] * gate[t, h] * scale; ``out`` [T, heads * dv] may be a column range of a
    wider tensor (rows strided)."""
    _need_cuda(attended, gate, out, segment_of_token)
    tokens, heads, dv = attended.shape
    assert attended.is_contiguous() and out.shape == (tokens, heads * dv) and out.stride(1) == 1
    assert gate is None or (gate.dtype == torch.float32 and gate.shape == (tokens, heads) and gate.is_contiguous())
    check(library.load().lse_head_gate_scale(attended.data_ptr(), dtype_code(attended.dtype), _ptr(gate), out.data_ptr(),
                                             dtype_code(out.dtype), out.stride(0), tokens, heads, dv, float(scale),
                                             _ptr(segment_of_token), _stream()), "head_gate_scale")
    return out


# ------------------------------------------------------------------ selective state-space scan
SELECTIVE_SCAN_CHUNK = 64          # rows of a chunk when a step's rows are scanned in chunks
SELECTIVE_SCAN_CHUNKED_FROM = 128  # rows of a step from which they are


def ssm_step_sizes(low: torch.Tensor, weight_t: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """dt float32 [T, C] = softplus(low[:, :rank] @ weight_t + bias); ``low``: a projection's rows (or partial sums),
    ``weight_t`` float32 [rank, C]."""
    _need_cuda(low, weight_t, bias)
    low, code, n_partials, stride, ld = _projection(low)
    tokens = low.shape[-2]
    rank, channels = weight_t.shape
    assert weight_t.dtype == bias.dtype == torch.float32 and weight_t.is_contiguous() and bias.shape == (channels,)
    assert low.shape[-1] >= rank
    dt = torch.empty((tokens, channels), dtype=torch.float32, device=low.device)
    check(library.load().lse_ssm_step_sizes(low.data_ptr(), code, n_partials, stride, ld, weight_t.data_ptr(),
                                            bias.data_ptr(), dt.data_ptr(), tokens, channels, rank, _stream()),
          "ssm_step_sizes")
    return dt


def selective_scan(x: torch.Tensor, dt: torch.Tensor, proj: torch.Tensor, z_off: int, low: torch.Tensor, b_off: int,
                   c_off: int, a_log: torch.Tensor, skip: torch.Tensor, state: torch.Tensor, step, out: torch.Tensor,
                   scale: float = 1.0, chunked: bool | None = None) -> torch.Tensor:
    """S[c, n] <- exp(dt[c] A[c, n]) S[c, n] + dt[c] x[c] B[n];  y[c] = sum_n S[c, n] C[n] + skip[c] x[c];
    out[t, c] = y[c] silu(z[c]) * scale, over the rows of every request in order, from and into ``state`` float32
    [slots, C, N].  A = -exp(a_log) (float32 [C, N]); B and C are columns b_off .. and c_off .. of ``low``, z columns
    z_off .. of ``proj`` (each a projection's rows or partial sums); x [T, C] in the compute dtype, dt float32 [T, C];
    ``out`` [T, C] may be a column range of a wider tensor.  ``chunked`` (default: from ``SELECTIVE_SCAN_CHUNKED_FROM``
    rows on): the rows of a request are cut into chunks that are scanned side by side, each from zero, then carried
    (a chunk's decay is exp(A * the sum of its step sizes)), then scanned again for the outputs."""
    _need_cuda(x, dt, proj, low, a_log, skip, state, out)
    proj, p_code, p_partials, p_stride, p_ld = _projection(proj)
    low, l_code, l_partials, l_stride, l_ld = _projection(low)
    tokens, channels = x.shape
    states = a_log.shape[1]
    assert x.is_contiguous() and dt.dtype == torch.float32 and dt.is_contiguous() and dt.shape == x.shape
    assert a_log.dtype == skip.dtype == torch.float32 and a_log.shape == (channels, states) and a_log.is_contiguous()
    assert skip.shape == (channels,)
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (channels, states)
    assert out.shape == (tokens, channels) and out.stride(1) == 1 and out.dtype == x.dtype
    chunk_rows, chunk_state, chunk_dt, max_chunks = 0, None, None, 0
    if chunked if chunked is not None else tokens >= SELECTIVE_SCAN_CHUNKED_FROM:
        chunk_rows = SELECTIVE_SCAN_CHUNK
        max_chunks = tokens // chunk_rows + step.segment_state_slot.shape[0]
        chunk_state = torch.empty((max_chunks, channels, states), dtype=torch.float32, device=out.device)
        chunk_dt = torch.empty((max_chunks, channels), dtype=torch.float32, device=out.device)
    check(library.load().lse_selective_scan(
        x.data_ptr(), dtype_code(x.dtype), dt.data_ptr(), proj.data_ptr(), p_code, p_partials, p_stride, p_ld, int(z_off),
        low.data_ptr(), l_code, l_partials, l_stride, l_ld, int(b_off), int(c_off), a_log.data_ptr(), skip.data_ptr(),
        state.data_ptr(), step.segment_start.data_ptr(), step.segment_state_slot.data_ptr(), out.data_ptr(),
        dtype_code(out.dtype), out.stride(0), float(scale), step.segment_state_slot.shape[0], channels, states,
        state.shape[0], chunk_rows, _ptr(chunk_state), _ptr(chunk_dt), max_chunks, _stream()), "selective_scan")
    return out
