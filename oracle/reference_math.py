"""CPU restatement of the reference arithmetic for the DiT attention path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module;
it is the checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline legs of ``bench.py``.

Every function restates, on CPU tensors, what the ``ref_program`` of one
reference kernel computes (file:line given per function, paths relative to the
reference project).  Pinning: ``tests/golden/make_golden.py`` imports the real
reference, runs its ``ref_program``s on CPU and stores their outputs; the test
``tests/test_oracle_golden.py`` checks these functions against those outputs
bit for bit (integer/byte tensors) or to 1e-6 (fp32 attention outputs).

Not pinned by the reference ("parity unpinned", there is nothing in the reference
to compare with): the Walsh-Hadamard rotation, the canonical summation order of
``token_group_mean`` (the reference sums in torch's own order; this module fixes
one and checks closeness to torch), 128-token int8 blocks are pinned through the
reference's generic formula.
"""

from __future__ import annotations


import numpy as np
import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
V_PERMUTATION = (0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15)
MEAN_CHUNK = 128
INV_SQRT_128 = np.float32(0.08838834764831845)


# ------------------------------------------------------------------ rotation
def hadamard128(values: torch.Tensor) -> torch.Tensor:
    """Normalised 128-point Walsh-Hadamard transform over the last axis (fp32).

    Sylvester order, evaluated as the butterfly network with strides 1,2,...,64
    (``x[i], x[i+h] = x[i]+x[i+h], x[i]-x[i+h]``), then multiplied by
    fl32(1/sqrt(128)).  No counterpart in the reference's attention path
    (its only Hadamard is the linear-layer ConvRot,
    src/nano_omni/kernels/quantization/convrot_int8.py:62-76): parity unpinned.
    """
    x = values.detach().to(torch.float32).numpy().copy()
    assert x.shape[-1] == 128
    h = 1
    while h < 128:
        y = x.reshape(*x.shape[:-1], 128 // (2 * h), 2, h)
        a = y[..., 0, :].copy()
        b = y[..., 1, :].copy()
        y[..., 0, :] = a + b
        y[..., 1, :] = a - b
        h *= 2
    return torch.from_numpy(x * INV_SQRT_128)


# --------------------------------------------------------------- column mean
def token_group_mean(source: torch.Tensor, tokens_per_block: int, include_padding: bool) -> torch.Tensor:
    """fp32 mean of bf16 rows per group of tokens.

    Semantics: src/nano_omni/kernels/normalization/token_group_mean.py:157-183
    (sum valid tokens, divide by the group size or by the valid count).  The
    reference leaves the summation order to torch; this restatement fixes it so
    that a GPU kernel can be bit-compared: chunks of 128 tokens summed
    sequentially in token order, chunk sums added sequentially in chunk order,
    one IEEE division at the end.
    """
    num_tokens, columns = source.shape
    x = source.to(torch.float32).numpy()
    groups = -(-num_tokens // tokens_per_block)
    out = np.zeros((groups, columns), dtype=np.float32)
    for g in range(groups):
        begin = g * tokens_per_block
        end = min(begin + tokens_per_block, num_tokens)
        total = None
        for c0 in range(begin, end, MEAN_CHUNK):
            c1 = min(c0 + MEAN_CHUNK, end)
            acc = np.zeros(columns, dtype=np.float32)
            for t in range(c0, c1):
                acc = acc + x[t]
            total = acc if total is None else total + acc
        divisor = np.float32(tokens_per_block if include_padding else end - begin)
        out[g] = total / divisor
    return torch.from_numpy(out)


# -------------------------------------------------------------- int8 Q and K
def int8_fp8_quantize_qk(
    source: torch.Tensor,
    statistics: torch.Tensor | None,
    heads: int,
    tokens_per_block: int,
    center: bool,
    hadamard: bool = False,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Symmetric int8 with one fp32 scale per (head, block of tokens).

    src/nano_omni/kernels/attention/int8_fp8/quantize_qk.py:170-201:
    x = f32(src) [- mean]; tokens zero-padded to whole blocks; scale =
    max(amax/127, 1e-10); q = clamp(round_half_even(x / scale), -128, 127);
    outputs head-major [heads, padded, 128] and [heads, blocks].
    """
    num_tokens = source.shape[0]
    x = source.to(torch.float32).reshape(num_tokens, heads, 128).clone()
    if center:
        x = x - statistics.reshape(1, heads, 128)
    if hadamard:
        x = hadamard128(x)
    blocks = -(-num_tokens // tokens_per_block)
    padded = blocks * tokens_per_block
    full = torch.zeros(padded, heads, 128, dtype=torch.float32)
    full[:num_tokens] = x
    grouped = full.reshape(blocks, tokens_per_block, heads, 128)
    amax = grouped.abs().amax(dim=(1, 3))  # [blocks, heads]
    scale = torch.clamp_min(amax / 127, 1e-10)
    q = torch.round(grouped / scale[:, None, :, None]).clamp(-128, 127).to(torch.int8)
    return q.permute(2, 0, 1, 3).reshape(heads, padded, 128).contiguous(), scale.T.contiguous()


# ------------------------------------------------------------------ fp8 V
def int8_fp8_value_scale(source: torch.Tensor, heads: int) -> torch.Tensor:
    """max(max_t |V| / 2.25, 1e-10) per (head, channel).

    src/nano_omni/kernels/attention/int8_fp8/value_scale.py:113-123.
    """
    amax = source.to(torch.float32).abs().amax(dim=0)
    return torch.clamp_min(amax / 2.25, 1e-10).reshape(heads, 128)


def int8_fp8_quantize_value(source: torch.Tensor, scale: torch.Tensor, heads: int) -> torch.Tensor:
    """V / scale -> e4m3, channel-major, tokens permuted inside groups of 16.

    src/nano_omni/kernels/attention/int8_fp8/quantize_value.py:136-152: stored
    position p of every 16-token group holds source token V_PERMUTATION[p];
    tokens are zero-padded to a multiple of 64.
    """
    num_tokens = source.shape[0]
    padded = -(-num_tokens // 64) * 64
    x = torch.zeros(padded, heads, 128, dtype=torch.float32)
    x[:num_tokens] = source.to(torch.float32).reshape(num_tokens, heads, 128)
    x = x / scale.reshape(1, heads, 128)
    order = torch.tensor(V_PERMUTATION)
    x = x.reshape(padded // 16, 16, heads, 128)[:, order].reshape(padded, heads, 128)
    return x.permute(1, 2, 0).contiguous().to(torch.float8_e4m3fn)


def unpermute_value_tokens(num_rows: int) -> torch.Tensor:
    """Index such that ``stored[..., index]`` lists tokens in logical order."""
    position = torch.arange(num_rows)
    logical = position // 16 * 16 + torch.tensor(V_PERMUTATION)[position % 16]
    return torch.argsort(logical)


# ------------------------------------------------------------------- NVFP4
def e2m1_codes(y: torch.Tensor) -> torch.Tensor:
    """Nearest e2m1 code (ties to the even code), sign in bit 3; input fp32."""
    a = y.abs()
    code = (
        (a > 0.25).to(torch.uint8)
        + (a >= 0.75).to(torch.uint8)
        + (a > 1.25).to(torch.uint8)
        + (a >= 1.75).to(torch.uint8)
        + (a > 2.5).to(torch.uint8)
        + (a >= 3.5).to(torch.uint8)
        + (a > 5.0).to(torch.uint8)
    )
    return code | (torch.signbit(y).to(torch.uint8) << 3)


def swizzle_scales(logical: torch.Tensor) -> torch.Tensor:
    """[heads, rows, groups] -> storage order in 512-byte atoms of 128 rows x 4 groups.

    src/nano_omni/kernels/attention/nvfp4_prepare.py:206-213: byte offset inside an
    atom = (r%32)*16 + (r%128//32)*4 + g%4; atoms row-block major, then group-block.
    """
    heads, rows, groups = logical.shape
    return (
        logical.reshape(heads, rows // 128, 4, 32, groups // 4, 4)
        .permute(0, 1, 4, 3, 2, 5)
        .contiguous()
        .reshape(heads, rows, groups)
    )


def unswizzle_scales(stored: torch.Tensor) -> torch.Tensor:
    heads, rows, groups = stored.shape
    return (
        stored.reshape(heads, rows // 128, groups // 4, 32, 4, 4)
        .permute(0, 1, 4, 3, 2, 5)
        .contiguous()
        .reshape(heads, rows, groups)
    )


def nvfp4_prepare(
    source: torch.Tensor,
    mean: torch.Tensor | None,
    heads: int,
    transpose: bool,
    hadamard: bool = False,
    global_scale: float = 0.0,
) -> tuple[torch.Tensor, torch.Tensor]:
    """e2m1 nibbles + one ue4m3 scale per 16 elements.

    global_scale == 0: src/nano_omni/kernels/attention/nvfp4_prepare.py:170-214
    (sf = e4m3(min(amax/6, 448)); y = x * (1/f32(sf)), 0 when sf == 0).
    global_scale > 0: src/nano_omni/kernels/quantization/quantize_fp4.py:221-262
    (bs = amax/(G*6) in fp32; y = x / (bs_or_1 * G); stored scale e4m3(bs)).
    Returns (packed u8 [heads, rows, cols/2], scales e4m3 bytes as uint8 in storage order).
    """
    num_tokens = source.shape[0]
    padded = -(-num_tokens // 128) * 128
    x = source.to(torch.float32).reshape(num_tokens, heads, 128)
    if mean is not None:
        x = x - mean[None]
    if hadamard:
        x = hadamard128(x)
    full = torch.zeros(padded, heads, 128, dtype=torch.float32)
    full[:num_tokens] = x
    full = full.permute(1, 2, 0) if transpose else full.permute(1, 0, 2)
    rows, cols = full.shape[1:]
    groups = full.reshape(heads, rows, cols // 16, 16)
    amax = groups.abs().amax(-1)
    if global_scale > 0:
        factor = torch.tensor(global_scale, dtype=torch.float32)
        block = amax / (factor * 6)
        safe = torch.where(block == 0, torch.ones_like(block), block)
        y = groups / (safe[..., None] * factor)
        stored = block.to(torch.float8_e4m3fn)
    else:
        stored = (amax / 6).clamp(max=448).to(torch.float8_e4m3fn)
        sf = stored.to(torch.float32)
        inverse = torch.where(sf == 0, torch.zeros_like(sf), 1.0 / sf)
        y = groups * inverse[..., None]
    codes = e2m1_codes(y).reshape(heads, rows, cols)
    packed = codes[..., 0::2] | (codes[..., 1::2] << 4)
    return packed.contiguous(), swizzle_scales(stored.view(torch.uint8))


def nvfp4_dequantize(packed: torch.Tensor, stored_scales: torch.Tensor) -> torch.Tensor:
    """Inverse of ``nvfp4_prepare`` (src/nano_omni/kernels/attention/dense_nvfp4.py:642-660)."""
    heads, rows, half = packed.shape
    cols = half * 2
    scales = unswizzle_scales(stored_scales.view(torch.uint8)).view(torch.float8_e4m3fn).to(torch.float32)
    codes = torch.stack((packed & 15, packed >> 4), dim=-1).reshape(heads, rows, cols).long()
    magnitude = torch.tensor(E2M1_VALUES, dtype=torch.float32)[codes & 7]
    values = torch.where(codes >= 8, -magnitude, magnitude)
    return values * scales.repeat_interleave(16, dim=-1)


# ---------------------------------------------------------------- attention
def dense_attention_fp32(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
    """softmax(Q K^T / sqrt(128)) V in fp32; inputs [tokens, heads, 128] any float dtype.

    The math of src/nano_omni/kernels/attention/dense_bf16.py:258-268 with the
    operands up-cast to fp32 (the accuracy target of the bf16 kernel).
    """
    q = query.to(torch.float32).transpose(0, 1)
    k = key.to(torch.float32).transpose(0, 1)
    v = value.to(torch.float32).transpose(0, 1)
    out = torch.nn.functional.scaled_dot_product_attention(q, k, v)
    return out.transpose(0, 1).contiguous()


def dense_bf16_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
    """The reference's own oracle: SDPA evaluated on the bf16 tensors as they are
    (src/nano_omni/kernels/attention/dense_bf16.py:258-268); result bf16."""
    out = torch.nn.functional.scaled_dot_product_attention(
        query.transpose(0, 1), key.transpose(0, 1), value.transpose(0, 1)
    )
    return out.transpose(0, 1).contiguous()


def int8_fp8_dequantize(query, key, value, query_scale, key_scale, value_scale, num_query_tokens: int, num_kv_tokens: int):
    """fp32 [heads, tokens, 128] operands from the int8 Q/K (scales per 32/64 tokens) and the
    e4m3 V (per-channel scale, tokens un-permuted): src/nano_omni/kernels/attention/int8_fp8/dense.py:394-420."""
    heads = query.shape[0]
    q = query.to(torch.float32).reshape(heads, -1, 32, 128) * query_scale[:, :, None, None]
    q = q.reshape(heads, -1, 128)[:, :num_query_tokens]
    k = key.to(torch.float32).reshape(heads, -1, 64, 128) * key_scale[:, :, None, None]
    k = k.reshape(heads, -1, 128)[:, :num_kv_tokens]
    order = unpermute_value_tokens(value.shape[2])[:num_kv_tokens]
    v = value.to(torch.float32)[:, :, order].transpose(1, 2) * value_scale[:, None, :]
    return q, k, v


def dense_int8_fp8_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    query_scale: torch.Tensor,
    key_scale: torch.Tensor,
    value_scale: torch.Tensor,
    num_query_tokens: int,
    num_kv_tokens: int,
) -> torch.Tensor:
    """Dequantise Q (32-token scales), K (64-token scales), V (per channel, tokens
    un-permuted) and evaluate fp32 attention per head.

    src/nano_omni/kernels/attention/int8_fp8/dense.py:394-437.  Returns bf16
    [num_query_tokens, heads*128].
    """
    heads = query.shape[0]
    q, k, v = int8_fp8_dequantize(query, key, value, query_scale, key_scale, value_scale, num_query_tokens, num_kv_tokens)
    out = torch.nn.functional.scaled_dot_product_attention(q, k, v)
    return out.transpose(0, 1).reshape(num_query_tokens, heads * 128).to(torch.bfloat16)


def dense_nvfp4_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    query_scales: torch.Tensor,
    key_scales: torch.Tensor,
    value_scales: torch.Tensor,
    num_query_tokens: int,
    num_kv_tokens: int,
) -> torch.Tensor:
    """Dequantise the three NVFP4 operands and evaluate fp32 attention.

    src/nano_omni/kernels/attention/dense_nvfp4.py:638-676.  Returns bf16
    [num_query_tokens, heads, 128].
    """
    q = nvfp4_dequantize(query, query_scales)[:, :num_query_tokens]
    k = nvfp4_dequantize(key, key_scales)[:, :num_kv_tokens]
    v = nvfp4_dequantize(value, value_scales).transpose(1, 2)[:, :num_kv_tokens]
    out = torch.nn.functional.scaled_dot_product_attention(q, k, v)
    return out.transpose(0, 1).contiguous().to(torch.bfloat16)


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.to(torch.float64).flatten()
    b = b.to(torch.float64).flatten()
    return float((a @ b) / (a.norm() * b.norm() + 1e-300))


def attention_flops(heads: int, num_query_tokens: int, num_kv_tokens: int) -> int:
    """Reference flop convention (src/nano_omni/kernels/attention/dense_bf16.py:252-255)."""
    return 4 * heads * num_query_tokens * num_kv_tokens * 128




# ------------------------------------------------------------------ norm + RoPE
def _row_inverse_rms(x: np.ndarray) -> np.ndarray:
    """1 / sqrt(sum(x^2) / 128 + 1e-5) per row of 128 with the summation order of the CUDA kernel:
    16 groups of 8 consecutive channels summed in channel order from 0, then an xor butterfly over the
    groups with strides 8, 4, 2, 1; every operation rounded to fp32."""
    f32 = np.float32
    sq = (x * x).astype(f32).reshape(*x.shape[:-1], 16, 8)
    part = np.zeros(sq.shape[:-1], dtype=f32)
    for i in range(8):
        part = (part + sq[..., i]).astype(f32)
    index = np.arange(16)
    for m in (8, 4, 2, 1):
        part = (part + part[..., index ^ m]).astype(f32)
    total = part[..., 0]
    root = np.sqrt((total * f32(0.0078125) + f32(1e-5)).astype(f32)).astype(f32)
    return (f32(1.0) / root).astype(f32)


def h3_head_norm_rope(
    source: torch.Tensor, weight: torch.Tensor, cosines: torch.Tensor | None, sines: torch.Tensor | None
) -> torch.Tensor:
    """Per-head RMS norm, optional split-half rotation of channel pairs (j, j + 48), bf16 result.

    src/nano_omni/kernels/specialized/h3_head_norm_rope.py:163-189 and h3_query_prepare.py:186-208
    (the two differ in how they sum the squares; the fixed order above stands for both).
    ``source`` bf16 [tokens, heads, 128]; ``cosines``/``sines`` f32 [tokens, 48].
    """
    f32 = np.float32
    x = source.to(torch.float32).numpy()
    w = weight.to(torch.float32).numpy()
    v = ((x * _row_inverse_rms(x)[..., None]).astype(f32) * w).astype(f32)
    if cosines is not None:
        c = cosines.numpy().astype(f32)[:, None, :]
        s = sines.numpy().astype(f32)[:, None, :]
        first, second = v[..., :48].copy(), v[..., 48:96].copy()
        v[..., :48] = ((first * c).astype(f32) - (second * s).astype(f32)).astype(f32)
        v[..., 48:96] = ((first * s).astype(f32) + (second * c).astype(f32)).astype(f32)
    return torch.from_numpy(v).to(torch.bfloat16)


def h3_query_prepare(
    source: torch.Tensor, weight: torch.Tensor, cosines: torch.Tensor | None, sines: torch.Tensor | None, heads: int
) -> tuple[torch.Tensor, torch.Tensor]:
    """Norm + rotation as above, then int8 with one scale per (head, 32 tokens)
    (src/nano_omni/kernels/specialized/h3_query_prepare.py:186-226)."""
    tokens = source.shape[0]
    rotated = h3_head_norm_rope(source.reshape(tokens, heads, 128), weight, cosines, sines)
    return int8_fp8_quantize_qk(rotated.reshape(tokens, heads * 128), None, heads, 32, False)


# ------------------------------------------------------------------ int8 GEMM
def matmul_int8(
    input: torch.Tensor,
    weight: torch.Tensor,
    weight_scale: torch.Tensor,
    input_scale: torch.Tensor,
    bias: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    multiply: torch.Tensor | None = None,
    use_silu: bool = False,
) -> torch.Tensor:
    """INT8 GEMM with the scaled fp32 epilogue, in the order of
    src/nano_omni/kernels/matmul/matmul_int8.py:229-240; exact int32 accumulation (int64 on CPU)."""
    value = (input.to(torch.int64) @ weight.to(torch.int64).T).to(torch.float32)
    value = value * weight_scale.reshape(1, -1)
    value = value * input_scale[:, None]
    if bias is not None:
        value = value + bias.float()
    if residual is not None:
        value = value + residual.float()
    if use_silu:
        value = torch.nn.functional.silu(value)
    if multiply is not None:
        value = value * multiply.float()
    return value.to(torch.bfloat16)


def matmul_bf16(
    input: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    multiply: torch.Tensor | None = None,
    output_scale: float = 1.0,
    use_silu: bool = False,
) -> torch.Tensor:
    """BF16 GEMM with the fp32 epilogue in the order of src/nano_omni/kernels/matmul/matmul_bf16.py:197-207.
    Accumulated in float64 here, so a tensor-core result (fp32, another summation order) agrees to fp32 rounding."""
    value = (input.double() @ weight.double().T).float()
    value = value * output_scale
    if bias is not None:
        value = value + bias.float()
    if residual is not None:
        value = value + residual.float()
    if use_silu:
        value = torch.nn.functional.silu(value)
    if multiply is not None:
        value = value * multiply.float()
    return value.to(torch.bfloat16)


def linear_int8(input, weight, weight_scale, *, bias=None, residual=None, multiply=None, use_silu=False, loras=(),
                rotation_group=0) -> torch.Tensor:
    """A projection with int8 weights as the reference operator chains it (src/nano_omni/ops/matmul/sequence.py:141-235):
    LoRA updates through the residual chain (each rounded to bf16), row-wise int8 activations, int8 GEMM."""
    for down, up, strength in loras:
        compressed = matmul_bf16(input, down)
        residual = matmul_bf16(compressed, up, None, residual, None, strength)
    quantized, scales = int8_rowwise(input, rotation_group)
    return matmul_int8(quantized, weight, weight_scale, scales, bias, residual, multiply, use_silu)


def _radix4(a, b, c, d):
    f32 = np.float32
    p, q, r, u = (a + b).astype(f32), (a - b).astype(f32), (c + d).astype(f32), (c - d).astype(f32)
    return (p + u).astype(f32), (p - u).astype(f32), (q + r).astype(f32), (r - q).astype(f32)


def convrot256(values: np.ndarray) -> np.ndarray:
    """Rotation of the last axis (256 columns) by B (x) B (x) B (x) B / 16, B the reference's 4 x 4 base matrix
    (src/nano_omni/kernels/quantization/convrot_int8.py:138-146), as four radix-4 stages over the base-4 digits of the
    column index, lowest digit first - the order of the CUDA kernel."""
    x = values.astype(np.float32).reshape(*values.shape[:-1], 4, 4, 4, 4)  # digits 3, 2, 1, 0
    for axis in (-1, -2, -3, -4):
        parts = [np.take(x, i, axis=axis) for i in range(4)]
        x = np.stack(_radix4(*parts), axis=axis)
    return (x.reshape(values.shape) * np.float32(0.0625)).astype(np.float32)


def int8_rowwise(source: torch.Tensor, rotation_group: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """Row-wise symmetric int8 in [-127, 127] with scale max(amax / 127, 1e-30)
    (src/nano_omni/kernels/quantization/int8_rowwise.py:107-116); with ``rotation_group`` 256 every group of 256
    columns is rotated and rounded to bf16 first (convrot_int8.py:130-161)."""
    values = source.to(torch.float32)
    if rotation_group:
        assert rotation_group == 256 and source.shape[1] % 256 == 0
        rotated = convrot256(values.numpy().reshape(source.shape[0], -1, 256)).reshape(source.shape)
        values = torch.from_numpy(rotated).to(torch.bfloat16).to(torch.float32)
    scale = torch.clamp_min(values.abs().amax(dim=1) / 127.0, 1e-30)
    quantized = torch.round(values / scale[:, None]).clamp_(-127, 127).to(torch.int8)
    return quantized, scale
