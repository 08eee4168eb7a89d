"""Exact stage (numerator + state) and finalize of the quantised sol paths on the GPU.

Checked against the CPU restatements of the reference ref_programs (oracle/sol_math.py, pinned to the
reference fixtures), against the reference outputs stored in the fixtures, and on the reference's own
known-answer cases (tests/test_sol_attention_state.py:231-460).  Tolerance of the final output is the
reference's rtol 0.02 / atol 0.02 (test_sol_attention_state.py:357, 455-459).
"""

import math

import pytest
import torch

from oracle import reference_math as rm
from oracle import sol_math as sm
from tests.conftest import bf16
from tests.gpu_util import desc, randn_bf16, run
from tests.test_gpu_attention_int8 import quantise
from tests.test_gpu_attention_nvfp4 import prepare
from tests.test_gpu_sol_route import gpu_pool, gpu_select, gpu_stats, structured_keys

pytestmark = pytest.mark.gpu


def int8_exact(ops, selected, T, h, total_heads=None, head_offset=0, protected=0):
    from nano_omni_b200.kernels.sol_exact import SolInt8Fp8AttentionArguments, SolInt8Fp8AttentionKernel

    q8, k8, v8, qs, ks, vs = ops
    H = total_heads or h
    exact = torch.full((T, H, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    state = torch.full((T, H, 2), float("nan"), device="cuda")
    run(
        SolInt8Fp8AttentionKernel(
            SolInt8Fp8AttentionArguments(
                desc(q8), desc(k8), desc(v8), desc(qs), desc(ks), desc(vs), desc(selected), desc(exact), desc(state),
                T, head_offset, 1.0, protected,
            )
        )
    )
    return exact, state


def nvfp4_exact(ops, selected, T, h, total_heads=None, head_offset=0, protected=1):
    from nano_omni_b200.core import DType
    from nano_omni_b200.kernels.sol_exact import SolNvfp4Arguments, SolNvfp4Kernel

    (q4, qsf), (k4, ksf), (v4, vsf) = ops
    H = total_heads or h
    exact = torch.full((T, H, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    state = torch.full((T, H, 2), float("nan"), device="cuda")
    u = DType.FP8_UE4M3
    run(
        SolNvfp4Kernel(
            SolNvfp4Arguments(
                desc(q4), desc(k4), desc(v4), desc(qsf, u), desc(ksf, u), desc(vsf, u), desc(selected), desc(exact),
                desc(state), T, T, head_offset, 1.0, protected,
            )
        )
    )
    return exact, state


def finalize(q, pooled3, selected, exact, state, head_offset=0, block=64, in_place=False):
    from nano_omni_b200.kernels.sol_exact import SolNvfp4FinalizeArguments, SolNvfp4FinalizeKernel

    out = exact if in_place else torch.full_like(exact, float("nan"))
    run(
        SolNvfp4FinalizeKernel(
            SolNvfp4FinalizeArguments(
                desc(q), desc(pooled3), desc(selected), desc(exact), desc(state), desc(out), head_offset, block
            )
        )
    )
    return out


def routed_case(T, h, seed, block=64):
    """bf16 inputs with block-structured keys, the three pooled planes and the routing mask, all from the GPU kernels."""
    q = randn_bf16(seed, T, h, 128)
    k = structured_keys(seed + 1, T, h, block)
    v = randn_bf16(seed + 2, T, h, 128)
    kmean = rm.token_group_mean(k.reshape(T, h * 128).cpu(), T, False).cuda()
    pooled3 = gpu_pool(k, v, kmean.reshape(h, 128).contiguous(), block)
    stats = gpu_stats(pooled3[0:2].contiguous())
    nb = -(-T // block)
    selected = gpu_select(q, pooled3[0].contiguous(), stats, 1.0, min(1, nb), block)
    return q, k, v, kmean, pooled3, selected


def numerator_error(got, want, want_state, rtol):
    """Largest excess of |got - want| over rtol*|want|, in units of sqrt(sum of probabilities) of the row.

    The numerator is a sum over the attended keys of rounded probabilities times values, so its rounding noise
    grows like the square root of the row's probability mass.
    """
    mass = want_state[..., 1:2].clamp(min=1.0).sqrt()
    return ((got - want).abs() - rtol * want.abs()) / mass


def check_state_and_numerator(exact, state, want_numerator, want_state, rtol, atol):
    got_state = state.cpu()
    torch.testing.assert_close(got_state[..., 0], want_state[..., 0], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(got_state[..., 1], want_state[..., 1], rtol=2e-3, atol=1e-4)
    got = exact.cpu().float()
    assert torch.isfinite(got).all()
    excess = numerator_error(got, want_numerator, want_state, rtol) - atol
    worst = int(excess.argmax())
    at = tuple(int(i) for i in torch.unravel_index(torch.tensor(worst), excess.shape))
    assert excess.max() <= 0, (
        f"numerator off at (token, head, channel) {at}: got {got[at]:.5f}, want {want_numerator[at]:.5f}, "
        f"state {got_state[at[0], at[1]].tolist()}; {int((excess > 0).sum())} elements over the bar"
    )


@pytest.mark.parametrize("T", [64, 65, 130, 300, 1000, 2100])
def test_int8_exact_stage_and_finalize_match_oracle(T):
    h = 2
    q, k, v, kmean, pooled3, selected = routed_case(T, h, 700 + T)
    flat = lambda t: t.reshape(T, h * 128)  # noqa: E731
    ops = quantise(flat(q), flat(k), flat(v), h)
    exact, state = int8_exact(ops, selected, T, h)
    dq, dk, dv = rm.int8_fp8_dequantize(*(t.cpu() for t in ops), T, T)
    want_numerator, want_state = sm.sol_exact_generic(
        dq, dk, dv, selected.cpu(), round_probability=sm.round_e4m3, probability_scale=448.0
    )
    # Probabilities are rounded to e4m3 relative to a maximum that the kernel raises lazily and the reference per
    # 64-key block, so the two round on different grids.  Both are measured against unrounded probabilities: the
    # kernel must stay within 0.1 * sqrt(mass) (the reference lands near 0.07) and within 1.5x the reference's own error.
    truth, _ = sm.sol_exact_generic(dq, dk, dv, selected.cpu())
    check_state_and_numerator(exact, state, truth, want_state, rtol=0.03, atol=0.1)
    mine = numerator_error(exact.cpu().float(), truth, want_state, 0.0).max()
    theirs = numerator_error(want_numerator, truth, want_state, 0.0).max()
    assert mine <= 1.5 * theirs + 1e-3, (float(mine), float(theirs))
    # finalize alone: same numerator and state into the oracle and the kernel
    out = finalize(q, pooled3, selected, exact, state)
    want = sm.sol_finalize(q.cpu(), pooled3.cpu(), selected.cpu(), exact.cpu(), state.cpu())
    torch.testing.assert_close(out.cpu().float(), want, rtol=0.02, atol=0.01)
    # the pair end to end: no further from the unrounded result than 1.5x the reference's rounding takes it
    final = lambda numerator: sm.sol_finalize(q.cpu(), pooled3.cpu(), selected.cpu(), numerator, want_state)  # noqa: E731
    true_end = final(truth)
    mine_end = (out.cpu().float() - true_end).abs().max()
    theirs_end = (final(want_numerator) - true_end).abs().max()
    assert mine_end <= 1.5 * theirs_end + 0.01, (float(mine_end), float(theirs_end))


@pytest.mark.parametrize("T", [65, 300, 1000])
def test_nvfp4_exact_stage_and_finalize_match_oracle(T):
    h = 2
    q, k, v, kmean, pooled3, selected = routed_case(T, h, 900 + T)
    flat = lambda t: t.reshape(T, h * 128).contiguous()  # noqa: E731
    ops = (
        prepare(flat(q), h, False),
        prepare(flat(k), h, False, kmean.reshape(h, 128).contiguous()),
        prepare(flat(v), h, True),
    )
    exact, state = nvfp4_exact(ops, selected, T, h)
    dq = rm.nvfp4_dequantize(ops[0][0].cpu(), ops[0][1].cpu())[:, :T]
    dk = rm.nvfp4_dequantize(ops[1][0].cpu(), ops[1][1].cpu())[:, :T]
    dv = rm.nvfp4_dequantize(ops[2][0].cpu(), ops[2][1].cpu()).transpose(1, 2)[:, :T]
    # Probabilities are rounded to e2m1 with a ue4m3 scale per 16 keys relative to a running maximum that kernel and
    # reference both raise per 64-key block; the kernel takes the union of two query blocks' lists and divides by an
    # approximate reciprocal of the scale, so single codes may round differently.  Both are measured against
    # unrounded probabilities: the kernel must stay within 1.5x the reference's own error.
    want_numerator, want_state = sm.sol_exact_generic(
        dq, dk, dv, selected.cpu(), always_first_block=True, round_probability=sm.round_nvfp4_groups, probability_scale=2688.0
    )
    truth, _ = sm.sol_exact_generic(dq, dk, dv, selected.cpu(), always_first_block=True)
    theirs = numerator_error(want_numerator, truth, want_state, 0.0).max()
    check_state_and_numerator(exact, state, truth, want_state, rtol=0.03, atol=float(1.5 * theirs + 1e-3))
    out = finalize(q, pooled3, selected, exact, state, in_place=True)
    true_end = sm.sol_finalize(q.cpu(), pooled3.cpu(), selected.cpu(), truth, want_state)
    mine_end = (out.cpu().float() - true_end).abs().max()
    theirs_end = (sm.sol_finalize(q.cpu(), pooled3.cpu(), selected.cpu(), want_numerator, want_state) - true_end).abs().max()
    assert mine_end <= 1.5 * theirs_end + 0.01, (float(mine_end), float(theirs_end))


def test_nvfp4_exact_stage_at_the_list_limit():
    """262144 keys = the 4096 list entries a query tile can hold, every block selected, fewer queries than keys.

    Size-independent properties: the state is the row maximum and the sum of unrounded probabilities of the dequantised
    operands; the normalised numerator is the dense result, where this kernel and the dense nvfp4 kernel (maximum raised
    per 64 and per 128 keys: different rounding grids for P) must be equally close to attention with unrounded P.
    """
    from tests.test_gpu_attention_nvfp4 import attend, dequantised

    Tq, Tk, h = 200, 4096 * 64, 1
    q = (randn_bf16(41, Tq, 128).float() * 2).bfloat16()
    k = randn_bf16(42, Tk, 128)
    v = randn_bf16(43, Tk, 128)
    ops = (prepare(q, h, False), prepare(k, h, False), prepare(v, h, True))
    selected = torch.ones((-(-Tq // 64), h, Tk // 64), dtype=torch.uint8, device="cuda")

    from nano_omni_b200.core import DType
    from nano_omni_b200.kernels.sol_exact import SolNvfp4Arguments, SolNvfp4Kernel

    (q4, qsf), (k4, ksf), (v4, vsf) = ops
    exact = torch.full((Tq, h, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    state = torch.full((Tq, h, 2), float("nan"), device="cuda")
    u = DType.FP8_UE4M3
    run(
        SolNvfp4Kernel(
            SolNvfp4Arguments(
                desc(q4), desc(k4), desc(v4), desc(qsf, u), desc(ksf, u), desc(vsf, u), desc(selected), desc(exact),
                desc(state), Tq, Tk, 0, 1.0, 1,
            )
        )
    )
    dense = attend(ops, Tq, h, Tk=Tk).float()

    dq, dk, dv = (t.cuda() for t in dequantised(ops, Tq, Tk))
    scores = torch.einsum("htd,hsd->hts", dq, dk)  # raw q.k
    top = scores.amax(-1)
    prob = torch.exp((scores - top[..., None]) / math.sqrt(128.0))
    truth = (torch.einsum("hts,hsd->htd", prob, dv) / prob.sum(-1, keepdim=True)).transpose(0, 1)
    assert torch.allclose(state[..., 0], top.transpose(0, 1), rtol=1e-5, atol=1e-5)
    assert torch.allclose(state[..., 1], prob.sum(-1).transpose(0, 1), rtol=2e-3)
    mine = exact.float() / state[..., 1:2]
    mine_err = (mine - truth).abs().max()
    dense_err = (dense - truth).abs().max()
    assert mine_err <= 1.5 * dense_err + 1e-3, (float(mine_err), float(dense_err))


def test_head_offset_block128_and_in_place_finalize():
    T, h, H, off, block = 700, 2, 5, 2, 128
    q, k, v, kmean, pooled3, selected = routed_case(T, h, 1234, block)
    from nano_omni_b200 import _lib
    import ctypes

    centred = (k.float() - kmean.reshape(1, h, 128)).bfloat16()
    exact = torch.full((T, H, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    state = torch.full((T, H, 2), 7.0, device="cuda")
    code = _lib.symbol("nob200_sol_exact_state_bf16_d128")(
        ctypes.c_int(T), ctypes.c_int(off), _lib.ptr(q), _lib.ptr(centred), _lib.ptr(v), _lib.ptr(selected),
        _lib.ptr(exact), _lib.ptr(state), ctypes.c_int(h), ctypes.c_int(H), ctypes.c_int(block), ctypes.c_int(0),
        ctypes.c_void_p(_lib.current_stream()),
    )
    assert code == 0, _lib.last_error()
    assert _lib.read_status() == 0
    hq, hk, hv = (t.cpu().float().transpose(0, 1) for t in (q, centred, v))
    want_numerator, want_state = sm.sol_exact_generic(hq, hk, hv, selected.cpu(), block=block)
    check_state_and_numerator(exact[:, off : off + h], state[:, off : off + h], want_numerator, want_state, 0.02, 0.02)
    assert (exact[:, :off] == 7).all() and (exact[:, off + h :] == 7).all()
    assert (state[:, :off] == 7).all() and (state[:, off + h :] == 7).all()
    want = sm.sol_finalize(
        q.cpu(), pooled3.cpu(), selected.cpu(), exact[:, off : off + h].cpu(), state[:, off : off + h].cpu(), block
    )
    out = finalize(q, pooled3, selected, exact, state, head_offset=off, block=block, in_place=True)
    assert out.data_ptr() == exact.data_ptr()
    torch.testing.assert_close(out[:, off : off + h].cpu().float(), want, rtol=0.02, atol=0.01)
    assert (out[:, :off] == 7).all() and (out[:, off + h :] == 7).all()


def test_rows_without_selected_blocks():
    """A query block that selects nothing: zeros and (-inf, 0) from the exact stage, pooled-only output after finalize."""
    T, h = 300, 2
    q, k, v, kmean, pooled3, selected = routed_case(T, h, 4321)
    selected = selected.clone()
    selected[1] = 0  # query block 1 (rows 64..127), both heads
    selected[3, 1] = 0
    flat = lambda t: t.reshape(T, h * 128)  # noqa: E731
    ops = quantise(flat(q), flat(k), flat(v), h)
    exact, state = int8_exact(ops, selected, T, h)
    assert (exact[64:128] == 0).all() and (exact[192:256, 1] == 0).all()
    assert torch.isinf(state[64:128, :, 0]).all() and (state[64:128, :, 0] < 0).all() and (state[64:128, :, 1] == 0).all()
    out = finalize(q, pooled3, selected, exact, state)
    want = sm.sol_finalize(q.cpu(), pooled3.cpu(), selected.cpu(), exact.cpu(), state.cpu())
    assert torch.isfinite(out.float()).all()
    torch.testing.assert_close(out.cpu().float(), want, rtol=0.02, atol=0.01)


def test_against_reference_fixtures(golden_sol):
    """Reference ref_program outputs: operands rebuilt by the (bit-exact) GPU quantisers from the fixture's bf16 inputs."""
    T, h, tag = 300, 2, "T300_h2"
    q, k, v = (bf16(golden_sol[f"{n}_{tag}"]).cuda() for n in "qkv")
    pooled3 = bf16(golden_sol[f"q_pooled3_{tag}"]).cuda()
    selected = torch.from_numpy(golden_sol[f"q_mask_{tag}"]).cuda()
    kmean = torch.from_numpy(golden_sol[f"q_kmean_{tag}"]).cuda()
    flat = lambda t: t.reshape(T, h * 128).contiguous()  # noqa: E731

    ops = quantise(flat(q), flat(k), flat(v), h)
    exact, state = int8_exact(ops, selected, T, h, protected=1)
    # the reference's numerator carries its own e4m3 rounding of the probabilities (another grid than the kernel's)
    check_state_and_numerator(
        exact, state, bf16(golden_sol[f"i8_exact_{tag}"]).float(), torch.from_numpy(golden_sol[f"i8_state_{tag}"]), 0.03, 0.15
    )
    out = finalize(q, pooled3, selected, exact, state)
    torch.testing.assert_close(out.cpu().float(), bf16(golden_sol[f"i8_final_{tag}"]).float(), rtol=0.02, atol=0.02)

    ops4 = (
        prepare(flat(q), h, False),
        prepare(flat(k), h, False, kmean.reshape(h, 128).contiguous()),
        prepare(flat(v), h, True),
    )
    exact4, state4 = nvfp4_exact(ops4, selected, T, h)
    # The reference rounds probabilities to e2m1 before the value product and so does the kernel, on another grid
    # (running maximum per 128-key tile instead of per 64-key block).  Same state; numerator and final output must
    # lie no further from the unrounded result than 1.5x the reference's.
    want_state4 = torch.from_numpy(golden_sol[f"f4_state_{tag}"])
    torch.testing.assert_close(state4.cpu(), want_state4, rtol=2e-3, atol=1e-4)
    dq = rm.nvfp4_dequantize(ops4[0][0].cpu(), ops4[0][1].cpu())[:, :T]
    dk = rm.nvfp4_dequantize(ops4[1][0].cpu(), ops4[1][1].cpu())[:, :T]
    dv = rm.nvfp4_dequantize(ops4[2][0].cpu(), ops4[2][1].cpu()).transpose(1, 2)[:, :T]
    truth, _ = sm.sol_exact_generic(dq, dk, dv, selected.cpu(), always_first_block=True)
    mine = numerator_error(exact4.cpu().float(), truth, want_state4, 0.0).max()
    theirs = numerator_error(bf16(golden_sol[f"f4_exact_{tag}"]).float(), truth, want_state4, 0.0).max()
    assert mine <= 1.5 * theirs + 1e-3, (float(mine), float(theirs))
    out4 = finalize(q, pooled3, selected, exact4, state4)
    true_end = sm.sol_finalize(q.cpu(), pooled3.cpu(), selected.cpu(), truth, want_state4)
    mine_end = (out4.cpu().float() - true_end).abs().max()
    theirs_end = (bf16(golden_sol[f"f4_final_{tag}"]).float() - true_end).abs().max()
    assert mine_end <= 1.5 * theirs_end + 0.01, (float(mine_end), float(theirs_end))


def test_int8_known_answer_raw_maximum_and_finalize():
    """tests/test_sol_attention_state.py:231-357: all-ones operands, 70 tokens, each block attends only itself."""
    T, nb = 70, 2
    ones = lambda *s, dtype: torch.ones(*s, dtype=dtype, device="cuda")  # noqa: E731
    ops = (
        ones(1, 96, 128, dtype=torch.int8), ones(1, 128, 128, dtype=torch.int8),
        torch.ones(1, 128, 128, device="cuda").to(torch.float8_e4m3fn),
        ones(1, 3, dtype=torch.float32), ones(1, 2, dtype=torch.float32), ones(1, 128, dtype=torch.float32),
    )  # fmt: skip
    selected = torch.zeros(nb, 1, nb, dtype=torch.uint8, device="cuda")
    selected[0, 0, 0] = 1
    selected[1, 0, 1] = 1
    exact, state = int8_exact(ops, selected, T, 1)
    torch.testing.assert_close(state[:, 0, 0].cpu(), torch.full((T,), 128.0))
    lengths = torch.tensor([64.0] * 64 + [6.0] * 6)
    torch.testing.assert_close(state[:, 0, 1].cpu(), lengths, rtol=1e-3, atol=0)
    torch.testing.assert_close(exact[:, 0].cpu().float(), lengths[:, None].expand(T, 128), rtol=2**-7, atol=0)

    pooled = torch.zeros(3, 1, nb, 128, dtype=torch.bfloat16, device="cuda")
    pooled[1].fill_(127 / 128)
    pooled[2, :, 0].fill_(128)
    pooled[2, :, 1].fill_(12)
    query = torch.ones(T, 1, 128, dtype=torch.bfloat16, device="cuda")
    out = finalize(query, pooled, selected, exact, state)
    scale = 128**-0.5
    score = float(query[0, 0].float() @ pooled[1, 0, 0].float())
    p = math.exp((score - 128.0) * scale)  # the pooled logit lies below the exact maximum
    expected = torch.empty(T)
    expected[:64] = (64.0 + p * 12.0) / (64.0 + p * 6.0)  # block 0 rows: pooled block 1 (6 tokens, V sum 12)
    expected[64:] = (6.0 + p * 128.0) / (6.0 + p * 64.0)  # block 1 rows: pooled block 0 (64 tokens, V sum 128)
    torch.testing.assert_close(out[:, 0].cpu().float(), expected[:, None].expand(T, 128), rtol=0.02, atol=0.02)


def test_nvfp4_known_answer_probability_units():
    """tests/test_sol_attention_state.py:360-460: all-ones nvfp4 operands, only key block 0 selected."""
    T, nb = 130, 3
    packed = torch.full((1, 256, 64), 0x22, dtype=torch.uint8, device="cuda")  # e2m1 code 2 = +1 in both nibbles
    packed_v = torch.full((1, 128, 128), 0x22, dtype=torch.uint8, device="cuda")
    one = torch.ones(1, dtype=torch.float32).to(torch.float8_e4m3fn).view(torch.uint8).item()
    scales = torch.full((1, 256, 8), one, dtype=torch.uint8, device="cuda")
    scales_v = torch.full((1, 128, 16), one, dtype=torch.uint8, device="cuda")
    selected = torch.zeros(nb, 1, nb, dtype=torch.uint8, device="cuda")
    selected[:, :, 0] = 1
    exact, state = nvfp4_exact(((packed, scales), (packed.clone(), scales.clone()), (packed_v, scales_v)), selected, T, 1)
    torch.testing.assert_close(state[:, 0, 0].cpu(), torch.full((T,), 128.0))
    torch.testing.assert_close(state[:, 0, 1].cpu(), torch.full((T,), 64.0))
    torch.testing.assert_close(exact[:, 0].cpu().float(), torch.full((T, 128), 64.0))

    query = torch.ones(T, 1, 128, dtype=torch.bfloat16, device="cuda")
    pooled = torch.zeros(3, 1, nb, 128, dtype=torch.bfloat16, device="cuda")
    pooled[1].fill_(1)
    for block, length in enumerate((64, 64, 2)):
        pooled[2, :, block].fill_(length * 2)
    out = finalize(query, pooled, selected, exact, state)
    expected = (64 + (64 + 2) * 2) / T  # equal logits everywhere: block 0 has V = 1, the pooled blocks V = 2
    torch.testing.assert_close(out.cpu().float(), torch.full((T, 1, 128), expected), rtol=0.02, atol=0.02)
