"""Paged-KV decode attention on the GPU against the CPU restatement of paged_kv_decode_attention_f32."""
import numpy as np
import pytest
import torch

from oracle import oracle
from singe_b200 import ops, workloads
from singe_b200 import kernel_sys as ks
from tests.gpu_util import assert_close_bf16, assert_close_f32, dev, dev_u32, host

pytestmark = pytest.mark.gpu


def _inputs(case, seed, bf16=True):
    rng = np.random.default_rng(seed)
    make = (lambda shape: workloads.normal_bf16(rng, shape)) if bf16 else (
        lambda shape: rng.standard_normal(shape, dtype=np.float32))
    q = make((case.batch, case.heads, case.head_dim))
    k = make((case.physical_blocks, case.block_size, case.kv_heads, case.head_dim))
    v = make((case.physical_blocks, case.block_size, case.kv_heads, case.head_dim))
    return q, k, v


def _config(case):
    return ops.PagedKvDecodeAttentionConfig.contiguous(case.batch, case.heads, case.kv_heads, case.head_dim,
                                                       case.block_size, case.physical_blocks,
                                                       case.block_table_batch_stride, case.scale)


def _oracle(case, q, k, v):
    return oracle.paged_kv_decode_attention_f32(
        q, k, v, case.lens, case.block_table, batch=case.batch, heads=case.heads, kv_heads=case.kv_heads,
        head_dim=case.head_dim, block_size=case.block_size, block_table_batch_stride=case.block_table_batch_stride,
        scale=case.scale)


def _decode(case, q, k, v, dtype):
    out = torch.full((case.batch, case.heads, case.head_dim), float("nan"), dtype=dtype, device="cuda")
    ops.paged_kv_decode_attention(out, dev(q, dtype), dev(k, dtype), dev(v, dtype), dev(case.lens),
                                  dev_u32(case.block_table), _config(case))
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    return host(out)


def test_config2_bf16_decode_matches_the_oracle():
    # 32 sequences, lengths U[128, 4096] (seed 1), 32 Q / 8 KV heads, head_dim 128, 16-token pages, +10 % pool.
    case = workloads.paged_decode_case()
    q, k, v = _inputs(case, seed=1)
    assert_close_bf16(_decode(case, q, k, v, torch.bfloat16), _oracle(case, q, k, v), "config 2 decode")


@pytest.mark.parametrize("lens", [[1], [15, 16, 17], [0, 33, 0, 512], [511, 512, 513, 1024, 1025], [4096, 7]])
@pytest.mark.parametrize("heads,kv_heads,head_dim", [(32, 8, 128), (8, 8, 128), (16, 2, 64), (4, 1, 128)])
def test_bf16_decode_edge_lengths_and_groupings(lens, heads, kv_heads, head_dim):
    case = workloads.paged_decode_case(seed=11, heads=heads, kv_heads=kv_heads, head_dim=head_dim, lens=lens)
    q, k, v = _inputs(case, seed=12)
    got = _decode(case, q, k, v, torch.bfloat16)
    ref = _oracle(case, q, k, v)
    assert_close_bf16(got, ref, f"lens={lens} heads={heads}/{kv_heads} d={head_dim}")
    for b, n in enumerate(lens):
        if n == 0:
            assert not got[b].any()  # an empty sequence writes zeros (cpu/attention.rs:1187,1211)


def test_f16_decode_matches_the_oracle():
    case = workloads.paged_decode_case(seed=21, lens=[100, 700, 2049])
    rng = np.random.default_rng(22)
    q, k, v = (rng.standard_normal(s).astype(np.float16).astype(np.float32) for s in (
        (case.batch, case.heads, case.head_dim),
        (case.physical_blocks, case.block_size, case.kv_heads, case.head_dim),
        (case.physical_blocks, case.block_size, case.kv_heads, case.head_dim)))
    assert_close_bf16(_decode(case, q, k, v, torch.float16), _oracle(case, q, k, v), "f16 decode")


@pytest.mark.parametrize("heads,kv_heads,head_dim,block_size", [(4, 2, 8, 4), (32, 8, 128, 16), (6, 3, 80, 8)])
def test_f32_decode_is_within_1e_4(heads, kv_heads, head_dim, block_size):
    case = workloads.paged_decode_case(seed=31, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                       block_size=block_size, lens=[5, 0, 129, 1000], max_len=1024)
    q, k, v = _inputs(case, seed=32, bf16=False)
    assert_close_f32(_decode(case, q, k, v, torch.float32), _oracle(case, q, k, v), "f32 decode")


def test_general_kernel_serves_shapes_the_tiled_kernel_does_not_take():
    # head_dim 96 and 32-token pages fall outside the tensor-core kernel; bf16 still within tolerance.
    case = workloads.paged_decode_case(seed=41, heads=8, kv_heads=4, head_dim=96, block_size=32, lens=[70, 300],
                                       max_len=512)
    q, k, v = _inputs(case, seed=42)
    assert_close_bf16(_decode(case, q, k, v, torch.bfloat16), _oracle(case, q, k, v), "general bf16 decode")


@pytest.mark.parametrize("max_splits", [1, 2, 4, 6, 64])
def test_caller_scratch_split_k_matches_for_every_split_budget(max_splits):
    # split ladders of the reference's own config tests: {1, 2, 4, 6} (singe-kernel/src/cuda/attention/tests.rs:128-190)
    case = workloads.paged_decode_case(seed=51, lens=[3000, 130, 16, 4096, 0, 777])
    q, k, v = _inputs(case, seed=52)
    out = torch.full((case.batch, case.heads, case.head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
    attn = torch.full((case.batch, case.heads, max_splits, case.head_dim), float("nan"), device="cuda")
    lse = torch.full((case.batch, case.heads, max_splits), float("nan"), device="cuda")
    ops.paged_kv_decode_splitk_reduce(out, attn, lse, dev(q, torch.bfloat16), dev(k, torch.bfloat16),
                                      dev(v, torch.bfloat16), dev(case.lens), dev_u32(case.block_table),
                                      _config(case), max_splits)
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    assert_close_bf16(host(out), _oracle(case, q, k, v), f"split-K decode, max_splits={max_splits}")


def test_partials_reduce_through_the_reference_combine():
    # Partials [B,H,S,D] + natural-log LSE [B,H,S]; both the device combine and the oracle's splitk_reduce_f32
    # (singe-kernel/src/cpu/attention.rs:2157-2193) must rebuild the unsplit result from them.
    case = workloads.paged_decode_case(seed=61, lens=[2048, 333, 4000])
    q, k, v = _inputs(case, seed=62)
    splits = 8
    attn = torch.full((case.batch, case.heads, splits, case.head_dim), float("nan"), device="cuda")
    lse = torch.full((case.batch, case.heads, splits), float("nan"), device="cuda")
    ops.paged_kv_decode_splitk(attn, lse, dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16),
                               dev(case.lens), dev_u32(case.block_table), _config(case), splits)
    out = torch.empty((case.batch, case.heads, case.head_dim), device="cuda")
    ops.splitk_reduce_f32(out, attn, lse, case.batch, case.heads, splits, case.head_dim)
    torch.cuda.synchronize()
    assert ops.take_device_error() == 0
    ref = _oracle(case, q, k, v)
    assert_close_bf16(host(out), ref, "device combine of device partials")
    cpu = oracle.splitk_reduce_f32(host(attn), host(lse), batch=case.batch, heads=case.heads, splits=splits,
                                   head_dim=case.head_dim)
    assert_close_bf16(cpu, ref, "oracle combine of device partials")
    assert_close_f32(host(out), cpu, "device combine vs oracle combine", 1e-5)
    per = ops.paged_kv_decode_split_tokens(case.block_table_batch_stride * case.block_size, splits, case.block_size)
    used = (case.lens + per - 1) // per
    for b in range(case.batch):
        assert np.isneginf(host(lse)[b, :, used[b]:]).all() and np.isfinite(host(lse)[b, :, :used[b]]).all()


def test_validation_mirrors_the_reference_config_checks():
    # validate_paged_kv_decode_attention_config (singe-kernel/src/cuda/attention/mod.rs:2963-2985)
    good = dict(batch=1, heads=4, kv_heads=2, head_dim=8, block_size=4, physical_blocks=2,
                block_table_batch_stride=2, scale=1.0)
    ops.PagedKvDecodeAttentionConfig.contiguous(**good)
    for field, value in [("batch", 0), ("heads", 0), ("kv_heads", 0), ("head_dim", 0), ("block_size", 0),
                         ("physical_blocks", 0), ("block_table_batch_stride", 0), ("heads", 3),
                         ("scale", float("inf")), ("scale", float("nan"))]:
        with pytest.raises(ops.SingeError) as caught:
            ops.PagedKvDecodeAttentionConfig.contiguous(**dict(good, **{field: value}))
        assert caught.value.code == ks.ERR_INVALID_LENGTH
    with pytest.raises(ops.SingeError) as caught:
        ops.PagedKvDecodeAttentionConfig.contiguous(**dict(good, batch=2**31))
    assert caught.value.code == ks.ERR_LENGTH_EXCEEDS_I32
    # the C ABI applies the same checks to raw calls
    lib = ks.lib()
    assert lib.singe_paged_kv_decode_attention_bf16(None, None, None, None, None, None, None, 1, 3, 2, 8, 4, 2, 2,
                                                    1.0) == ks.ERR_INVALID_LENGTH
    assert lib.singe_paged_kv_decode_attention_bf16(None, None, None, None, None, None, None, 1, 4, 2, 8, 4, 2, 2,
                                                    1.0) == ks.ERR_NULL_POINTER
    # buffers are "at least" sized: a short output is LengthTooShort
    case = workloads.paged_decode_case(seed=71, lens=[20])
    q, k, v = _inputs(case, seed=72)
    short = torch.empty(case.heads * case.head_dim - 1, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.SingeError) as caught:
        ops.paged_kv_decode_attention(short, dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16),
                                      dev(case.lens), dev_u32(case.block_table), _config(case))
    assert caught.value.code == ks.ERR_LENGTH_TOO_SHORT


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(32, 8, 128), (16, 2, 64)])
@pytest.mark.parametrize("normalise", [False, True])
@pytest.mark.parametrize("hinted", [False, True])
def test_decode_that_rotates_its_own_queries(heads, kv_heads, head_dim, normalise, hinted):
    # singe_rotary_paged_attention (kernel_plan/source/paged_attention.rs:535-542,881-977): the attention kernel takes the
    # query projections before the rotary embedding.  Without the norm the result must EQUAL the separate rotation
    # followed by the plain decode call (same rounding chain); with the per-head RMSNorm it is checked against the CPU
    # restatement: RmsNorm per head -> rotate_pairs -> paged_kv_decode_attention.
    from oracle import llama_ref
    from singe_b200.llama import rotary_tables

    lens = [1, 300, 16, 2049, 0, 777]
    case = workloads.paged_decode_case(seed=21, heads=heads, kv_heads=kv_heads, head_dim=head_dim, lens=lens)
    q, k, v = _inputs(case, seed=22)
    rng = np.random.default_rng(23)
    capacity, eps, splits = 4096, 1e-6, 6
    positions = np.array([0, 299, 15, 2048, 5, -1], dtype=np.int64)          # -1 wraps to capacity - 1
    cos, sin = rotary_tables(head_dim, 500000.0, capacity)
    gain = llama_ref.bf16(1.0 + 0.1 * rng.standard_normal(head_dim).astype(np.float32))
    lib = ks.lib()
    stream = int(torch.cuda.current_stream().cuda_stream)
    d_q, d_k, d_v = dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16)
    d_lens, d_table = dev(case.lens), dev_u32(case.block_table)
    d_cos, d_sin, d_positions = dev(cos, torch.bfloat16), dev(sin, torch.bfloat16), dev(positions)
    d_gain = dev(gain, torch.bfloat16)
    scratch = torch.empty((case.batch, heads, splits, head_dim + 1), dtype=torch.float32, device="cuda")
    attn_scratch, lse_scratch = scratch[..., :head_dim].contiguous(), scratch[..., head_dim].contiguous()
    out = torch.full((case.batch, heads, head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
    hints = ks.HINT_STABLE_PAGING if hinted else 0
    code = lib.singe_rotary_paged_kv_decode_attention_bf16(
        stream, out.data_ptr(), attn_scratch.data_ptr(), lse_scratch.data_ptr(), d_q.data_ptr(), d_k.data_ptr(),
        d_v.data_ptr(), d_lens.data_ptr(), d_table.data_ptr(), d_cos.data_ptr(), d_sin.data_ptr(),
        d_positions.data_ptr(), 8, case.batch, heads, kv_heads, head_dim, case.block_size, case.physical_blocks,
        case.block_table_batch_stride, splits, capacity, case.scale, int(normalise),
        d_gain.data_ptr() if normalise else None, eps, hints)
    torch.cuda.synchronize()
    assert code == ks.OK and ops.take_device_error() == 0
    wrapped = np.where(positions < 0, positions + capacity, positions)
    c, s = llama_ref.bf16(cos)[wrapped], llama_ref.bf16(sin)[wrapped]
    prepared = llama_ref.rms_norm(q.reshape(-1, head_dim), gain, eps).reshape(q.shape) if normalise else q
    rotated = llama_ref.rotate(prepared, c, s)
    assert_close_bf16(host(out), _oracle(case, rotated, k, v), "decode over queries rotated in the kernel")
    if not normalise:
        # the separate path: rotate on the host exactly as the rotary kernel rounds, then the plain split-K decode call
        separate = torch.full_like(out, float("nan"))
        code = lib.singe_paged_kv_decode_splitk_reduce_bf16(
            stream, separate.data_ptr(), attn_scratch.data_ptr(), lse_scratch.data_ptr(),
            dev(rotated, torch.bfloat16).data_ptr(), d_k.data_ptr(), d_v.data_ptr(), d_lens.data_ptr(),
            d_table.data_ptr(), case.batch, heads, kv_heads, head_dim, case.block_size, case.physical_blocks,
            case.block_table_batch_stride, splits, case.scale)
        torch.cuda.synchronize()
        assert code == ks.OK and torch.equal(out, separate)


@pytest.mark.parametrize("hinted", [False, True])
def test_the_last_split_of_a_row_folds_it_inside_the_decode_kernel(hinted):
    # With a ticket array the decode kernel needs no combine launch: whichever split of a (sequence, KV head) row
    # finishes last reads the row's partials back and writes the row, with the combine kernel's arithmetic -- so the
    # result must EQUAL the two-launch path -- and leaves the tickets at zero for the next call.
    lens = [1, 300, 16, 2049, 0, 777, 4096, 513]
    case = workloads.paged_decode_case(seed=41, heads=16, kv_heads=4, head_dim=128, lens=lens)
    q, k, v = _inputs(case, seed=42)
    lib = ks.lib()
    stream = int(torch.cuda.current_stream().cuda_stream)
    d_q, d_k, d_v = dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(v, torch.bfloat16)
    d_lens, d_table = dev(case.lens), dev_u32(case.block_table)
    splits = 7
    attn = torch.empty((case.batch, case.heads, splits, case.head_dim), dtype=torch.float32, device="cuda")
    lse = torch.empty((case.batch, case.heads, splits), dtype=torch.float32, device="cuda")
    tickets = torch.zeros(case.batch * case.kv_heads, dtype=torch.int32, device="cuda")
    hints = ks.HINT_STABLE_PAGING if hinted else 0

    def run(out, with_tickets):
        return lib.singe_paged_kv_decode_step_bf16(
            stream, out.data_ptr(), attn.data_ptr(), lse.data_ptr(), d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr(),
            d_lens.data_ptr(), d_table.data_ptr(), case.batch, case.heads, case.kv_heads, case.head_dim,
            case.block_size, case.physical_blocks, case.block_table_batch_stride, splits, case.scale, hints,
            tickets.data_ptr() if with_tickets else None)

    two_launches = torch.full((case.batch, case.heads, case.head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert run(two_launches, False) == ks.OK
    torch.cuda.synchronize()
    for _ in range(3):   # repeated calls: the tickets reset themselves
        folded = torch.full_like(two_launches, float("nan"))
        assert run(folded, True) == ks.OK
        torch.cuda.synchronize()
        assert torch.equal(folded, two_launches)
        assert int(tickets.abs().sum().item()) == 0
    assert ops.take_device_error() == 0
    assert_close_bf16(host(two_launches), _oracle(case, q, k, v), "decode with a split budget of 7")


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(32, 8, 128), (16, 2, 64), (4, 4, 128)])
@pytest.mark.parametrize("hinted,folded", [(False, False), (True, True)])
def test_the_fused_decode_step_attention_equals_rotation_cache_write_and_decode(heads, kv_heads, head_dim, hinted, folded):
    # singe_decode_step_attention_bf16: rotary embedding of Q and of the new K, the slot-mapped write of the new K / V rows
    # and paged attention over cached + new keys in one launch, against the three-kernel chain it replaces (rotation
    # + cache write kernel, then the split-K decode): caches bit-identical, outputs within the bf16 tolerance of each
    # other and of the CPU restatement (the new key's score is summed in another order).
    from oracle import llama_ref
    from singe_b200.llama import rotary_tables

    lens = [1, 300, 16, 2049, 17, 777, 512, 513]     # lengths INCLUDING the new token: the last key's position + 1
    case = workloads.paged_decode_case(seed=51, heads=heads, kv_heads=kv_heads, head_dim=head_dim, lens=lens)
    _, k, v = _inputs(case, seed=52)
    rng = np.random.default_rng(53)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = workloads.normal_bf16(rng, (case.batch, width + 8))[:, :width]      # a row stride wider than the row
    capacity, splits = 4096, 6
    positions = np.asarray(lens, dtype=np.int64) - 1
    write_pages = np.asarray([case.block_table[b, (n - 1) // 16] for b, n in enumerate(lens)], dtype=np.int64)
    write_slots = (positions % 16).astype(np.int64)
    cos, sin = rotary_tables(head_dim, 500000.0, capacity)
    lib = ks.lib()
    stream = int(torch.cuda.current_stream().cuda_stream)
    d_qkv_full = dev(np.pad(qkv, ((0, 0), (0, 8))), torch.bfloat16)
    d_lens, d_table = dev(case.lens), dev_u32(case.block_table)
    d_cos, d_sin = dev(cos, torch.bfloat16), dev(sin, torch.bfloat16)
    d_positions, d_pages, d_slots = dev(positions), dev(write_pages), dev(write_slots)
    attn = torch.empty((case.batch, heads, splits, head_dim), dtype=torch.float32, device="cuda")
    lse = torch.empty((case.batch, heads, splits), dtype=torch.float32, device="cuda")
    tickets = torch.zeros(case.batch * kv_heads, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    hints = ks.HINT_STABLE_PAGING if hinted else 0
    # fused
    fused_k, fused_v = dev(k, torch.bfloat16), dev(v, torch.bfloat16)
    fused_out = torch.full((case.batch, heads, head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
    code = lib.singe_decode_step_attention_bf16(
        stream, fused_out.data_ptr(), attn.data_ptr(), lse.data_ptr(), d_qkv_full.data_ptr(), width + 8,
        fused_k.data_ptr(), fused_v.data_ptr(), d_lens.data_ptr(), d_table.data_ptr(), d_cos.data_ptr(),
        d_sin.data_ptr(), d_positions.data_ptr(), d_pages.data_ptr(), d_slots.data_ptr(), 8, case.batch, heads,
        kv_heads, head_dim, 16, case.physical_blocks, case.block_table_batch_stride, splits, capacity, case.scale,
        hints, tickets.data_ptr() if folded else None, status.data_ptr())
    torch.cuda.synchronize()
    assert code == ks.OK and int(status.item()) == 0 and ops.take_device_error() == 0
    # the chain it replaces
    chain_k, chain_v = dev(k, torch.bfloat16), dev(v, torch.bfloat16)
    rotated_q = torch.empty((case.batch, heads, head_dim), dtype=torch.bfloat16, device="cuda")
    assert lib.singe_rotary_cache_write_bf16(
        stream, rotated_q.data_ptr(), d_qkv_full.data_ptr(), width + 8, d_cos.data_ptr(), d_sin.data_ptr(),
        d_positions.data_ptr(), chain_k.data_ptr(), chain_v.data_ptr(), d_pages.data_ptr(), d_slots.data_ptr(), 8,
        case.batch, heads, kv_heads, head_dim, case.physical_blocks, 16, capacity, status.data_ptr()) == ks.OK
    chain_out = torch.full_like(fused_out, float("nan"))
    assert lib.singe_paged_kv_decode_splitk_reduce_bf16(
        stream, chain_out.data_ptr(), attn.data_ptr(), lse.data_ptr(), rotated_q.data_ptr(), chain_k.data_ptr(),
        chain_v.data_ptr(), d_lens.data_ptr(), d_table.data_ptr(), case.batch, heads, kv_heads, head_dim, 16,
        case.physical_blocks, case.block_table_batch_stride, splits, case.scale) == ks.OK
    torch.cuda.synchronize()
    assert torch.equal(fused_k, chain_k) and torch.equal(fused_v, chain_v)     # the same rows in the same slots
    assert_close_bf16(host(fused_out), host(chain_out), "fused step attention vs the three-kernel chain")
    assert_close_bf16(host(fused_out), _oracle(case, host(rotated_q), host(chain_k), host(chain_v)),
                      "fused step attention vs the CPU restatement")
    assert int(tickets.abs().sum().item()) == 0
