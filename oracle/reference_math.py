"""CPU oracle: a numpy restatement of the reference's arithmetic for the quantized-GEMM path.

THIS IS TEST INFRASTRUCTURE.  Only the tests, the smoke check and the benchmark's CPU-baseline
leg may import it.  Nothing in the shipped package does, and nothing here is ever used to
produce a result handed to a user.

Parity status: PINNED.  ``tests/test_oracle.py`` checks every function here against
(1) the known-answer vectors of the reference's own tests (cited per function) and
(2) fixtures under ``tests/golden/`` produced by running the reference package itself
(``tests/golden/make_fixtures.py``).

Conventions: operands are numpy integer arrays; bf16 tensors travel as ``uint16`` bit patterns
(see :func:`bf16_bits_to_f32` / :func:`f32_to_bf16_bits`); results are float32 arrays whose
values are exactly the bf16 (or fp32) numbers the reference would store.

Integer matmul engine: ``float64`` BLAS.  Every product is an integer < 2**14 and every partial
sum is < 2**53, so the float64 result is the exact int32 accumulator of the reference's
``torch.matmul`` on int32 (api.py:304, :319); :func:`exact_int_matmul` can also run the int32
``torch.matmul`` itself (``engine="torch_int32"``), which is what the CPU baseline times.
"""
from __future__ import annotations

import numpy as np

LAYOUTS = ("nn", "nt", "tn", "tt")


# ----------------------------------------------------------------------------------------------
# bf16 <-> fp32
# ----------------------------------------------------------------------------------------------
def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 patterns -> float32 values (exact: bf16 is the top half of fp32)."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 patterns, round-to-nearest-even (what ``Tensor.to(torch.bfloat16)`` does)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    rounded = np.where(nan, (u >> 16) | 0x0040, rounded)
    return rounded.astype(np.uint16)


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bf16 value, returned as float32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# ----------------------------------------------------------------------------------------------
# operand format (reference quant.py)
# ----------------------------------------------------------------------------------------------
def fake_quant_int(x: np.ndarray, *, bits: int, scale: float) -> np.ndarray:
    """quant.py:14-29: ``clamp(round(float32(x) / scale), qmin, qmax)`` as int8, round-half-even."""
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    if scale <= 0:
        raise ValueError("scale must be positive")
    hi = (1 << (bits - 1)) - 1
    q = np.rint(np.asarray(x, dtype=np.float32) / np.float32(scale))
    return np.clip(q, -hi - 1, hi).astype(np.int8)


def pack_int4_k_major(x: np.ndarray) -> np.ndarray:
    """quant.py:32-38: byte = (odd & 0xF) << 4 | (even & 0xF) along the last axis, odd K zero-padded."""
    x = np.asarray(x)
    if x.shape[-1] % 2:
        pad = [(0, 0)] * (x.ndim - 1) + [(0, 1)]
        x = np.pad(x, pad)
    v = x.astype(np.int16)
    return ((v[..., 0::2] & 0xF) | ((v[..., 1::2] & 0xF) << 4)).astype(np.uint8)


def unpack_int4_k_major(p: np.ndarray) -> np.ndarray:
    """quant.py:41-51: low nibble -> even index, high nibble -> odd index, values >= 8 wrap to v - 16."""
    p = np.asarray(p, dtype=np.uint8)
    out = np.empty((*p.shape[:-1], p.shape[-1] * 2), dtype=np.int8)
    lo = (p & 0xF).astype(np.int8)
    hi = (p >> 4).astype(np.int8)
    out[..., 0::2] = np.where(lo >= 8, lo - 16, lo)
    out[..., 1::2] = np.where(hi >= 8, hi - 16, hi)
    return out


def pack_rhs_subchannel_scales(b_scale: np.ndarray) -> np.ndarray:
    """quant.py:54-65: (..., N, S) -> (..., S, N) contiguous."""
    return np.ascontiguousarray(np.swapaxes(b_scale, -1, -2))


def logical_operands(a: np.ndarray, b: np.ndarray, *, int4: bool, layout: str) -> tuple[np.ndarray, np.ndarray]:
    """api.py:267-281: stored operands -> logical ``A[M, K]``, ``B[K, N]`` integer arrays.

    Packed nibbles always run along K, which is the last stored axis only for the forms
    ``A [M, Kb]`` and ``B [N, Kb]``; the other forms are transposed before and after unpacking.
    """
    if layout not in LAYOUTS:
        raise ValueError(f"unknown layout {layout}")
    a_t = layout in ("tn", "tt")
    b_t = layout in ("nt", "tt")
    if int4 and a.dtype == np.uint8:
        a = np.swapaxes(unpack_int4_k_major(np.swapaxes(a, -1, -2)), -1, -2) if a_t else unpack_int4_k_major(a)
    if int4 and b.dtype == np.uint8:
        b = unpack_int4_k_major(b) if b_t else np.swapaxes(unpack_int4_k_major(np.swapaxes(b, -1, -2)), -1, -2)
    if a_t:
        a = np.swapaxes(a, -1, -2)
    if b_t:
        b = np.swapaxes(b, -1, -2)
    return a, b


# ----------------------------------------------------------------------------------------------
# the GEMM math (reference api.py:257-325)
# ----------------------------------------------------------------------------------------------
def exact_int_matmul(a: np.ndarray, b: np.ndarray, *, engine: str = "f64") -> np.ndarray:
    """Exact integer ``A @ B`` as int64.  api.py:304 (``torch.matmul`` on int32 operands)."""
    if engine == "f64":
        return np.rint(a.astype(np.float64) @ b.astype(np.float64)).astype(np.int64)
    if engine == "torch_int32":
        import torch

        ta = torch.from_numpy(np.ascontiguousarray(a)).to(torch.int32)
        tb = torch.from_numpy(np.ascontiguousarray(b)).to(torch.int32)
        return torch.matmul(ta, tb).numpy().astype(np.int64)
    raise ValueError(f"unknown engine {engine}")


def _acc_to_f32(acc: np.ndarray) -> np.ndarray:
    # int32 -> float32 is round-to-nearest-even, like Tensor.to(torch.float32)
    return acc.astype(np.int32).astype(np.float32)


def scaled_matmul(
    a_q: np.ndarray,
    b_q: np.ndarray,
    a_scale_f32: np.ndarray | None,
    b_scale_f32: np.ndarray | None,
    *,
    subchannel: int = 0,
    engine: str = "f64",
) -> np.ndarray:
    """api.py:299-325.  Per-channel: ``(f32(acc) * sa[:, None]) * sb[None, :]``.  Subchannel ``S``:
    for K-groups in ascending order ``out += (f32(acc_g) * sa[:, g, None]) * sb[g][None, :]``,
    ``out`` starting at zero, the last group possibly short."""
    if subchannel == 0:
        out = _acc_to_f32(exact_int_matmul(a_q, b_q, engine=engine))
        if a_scale_f32 is not None:
            out = out * a_scale_f32[..., :, None]
        if b_scale_f32 is not None:
            out = out * b_scale_f32[..., None, :]
        return out.astype(np.float32)
    k = a_q.shape[-1]
    out = np.zeros((*a_q.shape[:-1], b_q.shape[-1]), dtype=np.float32)
    for g, k0 in enumerate(range(0, k, subchannel)):
        k1 = min(k0 + subchannel, k)
        part = _acc_to_f32(exact_int_matmul(a_q[..., k0:k1], b_q[..., k0:k1, :], engine=engine))
        if a_scale_f32 is not None:
            part = part * a_scale_f32[..., :, g, None]
        if b_scale_f32 is not None:
            part = part * b_scale_f32[..., g, :][..., None, :]
        out += part.astype(np.float32)
    return out


def apply_epilogue(out: np.ndarray, epilogue: str) -> np.ndarray:
    """api.py:283-291: SwiGLU ``up * (gate / (1 + exp(-gate)))`` over ``[up | gate]`` columns; ReLU^2."""
    if epilogue == "none":
        return out
    if epilogue == "relu2":
        r = np.maximum(out, np.float32(0))
        return (r * r).astype(np.float32)
    if epilogue == "swiglu":
        if out.shape[-1] % 2:
            raise ValueError("fused SwiGLU reference requires an even output dimension")
        d = out.shape[-1] // 2
        up, gate = out[..., :d], out[..., d:]
        with np.errstate(over="ignore"):  # exp(-gate) -> inf for very negative gates gives gate/inf = -0, as in torch
            return (up * (gate / (np.float32(1.0) + np.exp(-gate)))).astype(np.float32)
    raise ValueError(f"unknown epilogue {epilogue}")


def reference_mm(
    a: np.ndarray,
    b: np.ndarray,
    *,
    int4: bool,
    layout: str = "nn",
    a_scale_bits: np.ndarray | None = None,
    b_scale_bits: np.ndarray | None = None,
    subchannel: int = 0,
    epilogue: str = "none",
    out_bf16: bool = True,
    engine: str = "f64",
) -> np.ndarray:
    """api.py:257-296 end to end.  Scales arrive as bf16 bit patterns; the result is float32
    holding exactly the stored values (bf16-rounded when ``out_bf16``)."""
    a_q, b_q = logical_operands(a, b, int4=int4, layout=layout)
    sa = None if a_scale_bits is None else bf16_bits_to_f32(a_scale_bits)
    sb = None if b_scale_bits is None else bf16_bits_to_f32(b_scale_bits)
    out = apply_epilogue(scaled_matmul(a_q, b_q, sa, sb, subchannel=subchannel, engine=engine), epilogue)
    return round_to_bf16(out) if out_bf16 else out


def int32_accumulators(a: np.ndarray, b: np.ndarray, *, int4: bool, layout: str = "nn") -> np.ndarray:
    """The exact int32 accumulators ``A_q @ B_q`` (metadata.py:10 ``ACC_DTYPE = "int32"``)."""
    a_q, b_q = logical_operands(a, b, int4=int4, layout=layout)
    return exact_int_matmul(a_q, b_q).astype(np.int32)


# ----------------------------------------------------------------------------------------------
# grouped dots (reference tests/test_ragged_dot.py:19-117 are the only statement of this math)
# ----------------------------------------------------------------------------------------------
def calculate_group_info(group_sizes, tile: int, *, tid_size: int | None = None, align_tile: int = 8) -> dict:
    """ragged.py:201-323 in plain integer loops.

    ``start_g = sum(sizes[:g])``; ``aligned_g = floor(start_g / align) * align``;
    ``blocks_g = 0 if size_g == 0 else floor((end_g - aligned_g + tile - 1) / tile)``; block ``j`` of
    group ``g``: ``block_start = aligned_g + j * tile``, ``actual_start = max(block_start, start_g)``,
    ``actual_end = min(block_start + tile, end_g)``.
    """
    if tile <= 0 or align_tile <= 0 or tile % align_tile:
        raise ValueError("tile must be a positive multiple of a positive align_tile")
    rows = {name: [] for name in ("group_id", "block_start", "actual_start", "actual_end", "start_within_block", "actual_size")}
    start = 0
    for g, size in enumerate(int(max(0, s)) for s in group_sizes):
        end = start + size
        if size:
            aligned = (start // align_tile) * align_tile
            for j in range((end - aligned + tile - 1) // tile):
                block = aligned + j * tile
                lo, hi = max(block, start), min(block + tile, end)
                for name, value in zip(rows, (g, block, lo, hi, lo - block, max(hi - lo, 0))):
                    rows[name].append(value)
        start = end
    num_tasks = len(rows["group_id"])
    length = num_tasks if tid_size is None else tid_size
    if length < num_tasks:
        raise ValueError(f"tid_size must be at least {num_tasks}; got {length}")
    out = {name: np.array(vals + [0] * (length - num_tasks), dtype=np.int64) for name, vals in rows.items()}
    out["num_tasks"] = num_tasks
    return out


def ragged_fwd_logical(lhs: np.ndarray, rhs: np.ndarray, layout: str) -> tuple[np.ndarray, np.ndarray]:
    """Stored forward operands -> logical ``x [M, K]`` and ``w [G, K, N]`` (test_ragged_dot.py:55-66 inverted)."""
    a_t = layout in ("tn", "tt")
    b_t = layout in ("nt", "tt")
    x = np.swapaxes(unpack_int4_k_major(np.swapaxes(lhs, 0, 1)), 0, 1) if a_t else unpack_int4_k_major(lhs)
    if a_t:
        x = np.swapaxes(x, 0, 1)
    w = unpack_int4_k_major(rhs) if b_t else np.swapaxes(unpack_int4_k_major(np.swapaxes(rhs, 1, 2)), 1, 2)
    if b_t:
        w = np.swapaxes(w, 1, 2)
    return x, w


def ragged_dot_fwd(
    lhs: np.ndarray,
    rhs: np.ndarray,
    group_sizes,
    a_scale_bits: np.ndarray,
    b_scale_bits: np.ndarray,
    *,
    layout: str = "nn",
    subchannel: int = 0,
    out_bf16: bool = True,
) -> np.ndarray:
    """test_ragged_dot.py:19-32 (per-channel) and :35-52 (subchannel): rows of group ``g`` times ``w[g]``."""
    x, w = ragged_fwd_logical(lhs, rhs, layout)
    sa = bf16_bits_to_f32(a_scale_bits)
    sb = bf16_bits_to_f32(b_scale_bits)
    out = np.zeros((x.shape[0], w.shape[2]), dtype=np.float32)
    row = 0
    for g, size in enumerate(int(s) for s in group_sizes):
        nxt = row + size
        if size:
            out[row:nxt] = scaled_matmul(x[row:nxt], w[g], sa[row:nxt], sb[g], subchannel=subchannel)
        row = nxt
    return round_to_bf16(out) if out_bf16 else out


def ragged_bwd_logical(lhs: np.ndarray, rhs: np.ndarray, layout: str) -> tuple[np.ndarray, np.ndarray]:
    """Stored backward operands -> logical ``a [G, M, K]`` and ``b [G, K, N]`` (test_ragged_dot.py:69-81 inverted)."""
    a_t = layout in ("tn", "tt")
    b_t = layout in ("nt", "tt")
    a = np.swapaxes(unpack_int4_k_major(np.swapaxes(lhs, 1, 2)), 1, 2) if a_t else unpack_int4_k_major(lhs)
    if a_t:
        a = np.swapaxes(a, 1, 2)
    b = unpack_int4_k_major(rhs) if b_t else np.swapaxes(unpack_int4_k_major(np.swapaxes(rhs, 1, 2)), 1, 2)
    if b_t:
        b = np.swapaxes(b, 1, 2)
    return a, b


def ragged_dot_bwd(
    lhs: np.ndarray,
    rhs: np.ndarray,
    group_sizes,
    a_scale_bits: np.ndarray,
    b_scale_bits: np.ndarray,
    *,
    layout: str = "nn",
    subchannel: int = 0,
) -> np.ndarray:
    """test_ragged_dot.py:84-97 and :100-117: ``out[g] = a[g][:, :k_g] @ b[g][:k_g]`` scaled; fp32.

    Subchannel groups are cut at multiples of ``S`` and clipped to ``k_g`` (``k1 = min(k0 + S, k_g)``);
    groups that start at or beyond ``k_g`` contribute nothing.
    """
    a, b = ragged_bwd_logical(lhs, rhs, layout)
    sa = bf16_bits_to_f32(a_scale_bits)
    sb = bf16_bits_to_f32(b_scale_bits)
    out = np.zeros((a.shape[0], a.shape[1], b.shape[2]), dtype=np.float32)
    for g, kg in enumerate(int(s) for s in group_sizes):
        if kg:
            out[g] = scaled_matmul(a[g][:, :kg], b[g][:kg], sa[g], sb[g], subchannel=subchannel)
    return out


# ----------------------------------------------------------------------------------------------
# formats either side of the path that the reference only handles on the host
# ----------------------------------------------------------------------------------------------
def repack_tokens(packed: np.ndarray) -> np.ndarray:
    """Packed int4 ``[T, F/2]`` (features paired) -> ``[ceil(T/2), F]`` (tokens paired).

    What the reference's test helper does per group with ``pack_int4_k_major(x.T).T``
    (tests/test_ragged_dot.py:67-81), here for one flat token axis.
    """
    codes = unpack_int4_k_major(packed)                     # [T, F]
    return np.ascontiguousarray(pack_int4_k_major(np.ascontiguousarray(codes.T)).T)


def ragged_dot_bwd_flat(
    lhs_tokens: np.ndarray,
    rhs_tokens: np.ndarray,
    group_sizes,
    a_scale_bits: np.ndarray,
    b_scale_bits: np.ndarray,
) -> np.ndarray:
    """Grouped backward dot over flat token-packed operands: the math of test_ragged_dot.py:84-97 with the
    groups taken as consecutive token ranges of ``lhs [ceil(T/2), M]`` / ``rhs [ceil(T/2), N]``."""
    x = unpack_int4_k_major(np.ascontiguousarray(lhs_tokens.T)).T    # [T', M] codes, T' = 2 * ceil(T/2)
    dy = unpack_int4_k_major(np.ascontiguousarray(rhs_tokens.T)).T   # [T', N]
    sa = bf16_bits_to_f32(a_scale_bits)
    sb = bf16_bits_to_f32(b_scale_bits)
    sizes = [int(s) for s in group_sizes]
    out = np.zeros((len(sizes), x.shape[1], dy.shape[1]), dtype=np.float32)
    start = 0
    for g, size in enumerate(sizes):
        if size:
            out[g] = scaled_matmul(np.ascontiguousarray(x[start:start + size].T), dy[start:start + size], sa[g], sb[g])
        start += size
    return out


# ----------------------------------------------------------------------------------------------
# metric (reference benchmarking.py:104-111)
# ----------------------------------------------------------------------------------------------
def tops_for_runtime(m: int, n: int, k: int, runtime_ms: float) -> float:
    return 2.0 * m * n * k / (runtime_ms / 1.0e3) / 1.0e12
