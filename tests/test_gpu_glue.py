"""Decode-step glue kernels (embedding, add + RMSNorm, rotary + cache write, SwiGLU, argmax) against the CPU
restatement, on widths that take the 128-bit path and on odd widths that take the scalar path."""
import numpy as np
import pytest
import torch

from oracle import llama_ref, oracle
from singe_b200 import kernel_sys as ks
from singe_b200 import workloads
from singe_b200.llama import rotary_tables
from tests.gpu_util import assert_close_bf16, dev, host

pytestmark = pytest.mark.gpu


def _stream():
    return int(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("width", [4096, 72, 100, 18000])
def test_add_rms_norm(width):
    rng = np.random.default_rng(width)
    rows = 5
    hidden = workloads.normal_bf16(rng, (rows, width))
    delta = workloads.normal_bf16(rng, (rows, width))
    weight = llama_ref.bf16(1.0 + 0.1 * rng.standard_normal(width).astype(np.float32))
    d_hidden, d_normed = dev(hidden, torch.bfloat16), torch.empty((rows, width), dtype=torch.bfloat16, device="cuda")
    d_delta, d_weight = dev(delta, torch.bfloat16), dev(weight, torch.bfloat16)  # kept alive across the launches
    code = ks.lib().singe_add_rms_norm_bf16(_stream(), d_hidden.data_ptr(), d_delta.data_ptr(),
                                            d_normed.data_ptr(), d_weight.data_ptr(), rows, width, 1e-5)
    assert code == ks.OK
    summed = llama_ref.bf16(hidden + delta)
    assert np.array_equal(host(d_hidden), summed)          # the residual add is one bf16 rounding: bit-exact
    assert_close_bf16(host(d_normed), llama_ref.rms_norm(summed, weight, 1e-5), "normed")
    plain = torch.empty_like(d_normed)
    assert ks.lib().singe_add_rms_norm_bf16(_stream(), d_hidden.data_ptr(), None, plain.data_ptr(),
                                            d_weight.data_ptr(), rows, width, 1e-5) == ks.OK
    torch.cuda.synchronize()
    assert torch.equal(plain, d_normed)


@pytest.mark.parametrize("width", [14336, 40, 33])
def test_silu_mul(width):
    rng = np.random.default_rng(width)
    rows = 7
    fused = workloads.normal_bf16(rng, (rows, 2 * width), std=2.0)
    d_fused = dev(fused, torch.bfloat16)
    out = torch.empty((rows, width), dtype=torch.bfloat16, device="cuda")
    assert ks.lib().singe_silu_mul_bf16(_stream(), out.data_ptr(), d_fused.data_ptr(),
                                        d_fused.data_ptr() + 2 * width, 2 * width, rows, width) == ks.OK
    assert_close_bf16(host(out), llama_ref.silu_mul(fused[:, :width], fused[:, width:]), "swiglu")


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(8, 2, 128), (4, 2, 16), (3, 1, 6)])
def test_rotary_cache_write(heads, kv_heads, head_dim):
    rng = np.random.default_rng(head_dim)
    tokens, pages, page_size, capacity = 6, 5, 4, 64
    qkv = workloads.normal_bf16(rng, (tokens, (heads + 2 * kv_heads) * head_dim))
    positions = np.array([0, 1, 17, 63, -1, 5], dtype=np.int64)  # -1 wraps to capacity - 1
    write_pages = np.array([0, 4, 2, -1, 1, 3], dtype=np.int64)
    write_slots = np.array([0, 3, -1, 1, 2, 0], dtype=np.int64)
    cos, sin = rotary_tables(head_dim, 500000.0, capacity)
    key_cache = workloads.normal_bf16(rng, (pages, page_size, kv_heads, head_dim))
    value_cache = workloads.normal_bf16(rng, (pages, page_size, kv_heads, head_dim))
    d_k, d_v = dev(key_cache, torch.bfloat16), dev(value_cache, torch.bfloat16)
    q_out = torch.empty((tokens, heads, head_dim), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    d_qkv = dev(qkv, torch.bfloat16)
    cos_d, sin_d = dev(cos, torch.bfloat16), dev(sin, torch.bfloat16)
    d_positions, d_pages, d_slots = dev(positions), dev(write_pages), dev(write_slots)
    code = ks.lib().singe_rotary_cache_write_bf16(
        _stream(), q_out.data_ptr(), d_qkv.data_ptr(), qkv.shape[1], cos_d.data_ptr(), sin_d.data_ptr(),
        d_positions.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), d_pages.data_ptr(), d_slots.data_ptr(), 8, tokens,
        heads, kv_heads, head_dim, pages, page_size, capacity, status.data_ptr())
    torch.cuda.synchronize()
    assert code == ks.OK and int(status.item()) == 0
    wrapped = np.where(positions < 0, positions + capacity, positions)
    c, s = llama_ref.bf16(cos)[wrapped], llama_ref.bf16(sin)[wrapped]
    q = qkv[:, : heads * head_dim].reshape(tokens, heads, head_dim)
    k = qkv[:, heads * head_dim: (heads + kv_heads) * head_dim].reshape(tokens, kv_heads, head_dim)
    v = qkv[:, (heads + kv_heads) * head_dim:].reshape(tokens, kv_heads, head_dim)
    assert np.array_equal(host(q_out), llama_ref.rotate(q, c, s))      # the rounding chain is reproduced: bit-exact
    expect_k, expect_v = key_cache.copy(), value_cache.copy()
    assert oracle.kv_cache_write(expect_k, np.ascontiguousarray(llama_ref.rotate(k, c, s)), write_pages,
                                 write_slots) == oracle.OK
    assert oracle.kv_cache_write(expect_v, np.ascontiguousarray(v), write_pages, write_slots) == oracle.OK
    assert np.array_equal(host(d_k), expect_k) and np.array_equal(host(d_v), expect_v)
    # a slot outside the cache is dropped and reported; the queries are still rotated
    bad_pages = write_pages.copy()
    bad_pages[2] = pages
    d_bad = dev(bad_pages)
    code = ks.lib().singe_rotary_cache_write_bf16(
        _stream(), q_out.data_ptr(), d_qkv.data_ptr(), qkv.shape[1], cos_d.data_ptr(), sin_d.data_ptr(),
        d_positions.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), d_bad.data_ptr(), d_slots.data_ptr(), 8, tokens,
        heads, kv_heads, head_dim, pages, page_size, capacity, status.data_ptr())
    torch.cuda.synchronize()
    assert code == ks.OK and int(status.item()) == 1
    assert np.array_equal(host(d_k), expect_k)


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(8, 2, 128), (4, 2, 16), (2, 1, 64)])
@pytest.mark.parametrize("which", ["both", "query with a gain", "key without a gain"])
def test_rotary_cache_write_with_per_head_rms_norm(heads, kv_heads, head_dim, which):
    # query_norm / key_norm of the reference's fused kernel (kernel_plan/source/rotary_cache.rs:25-52): RmsNorm over
    # each head, rounded to bf16 as the separate op returns it, then the rotation's rounding chain
    rng = np.random.default_rng(head_dim + len(which))
    tokens, pages, page_size, capacity, eps = 5, 4, 4, 32, 1e-6
    qkv = workloads.normal_bf16(rng, (tokens, (heads + 2 * kv_heads) * head_dim))
    positions = np.array([0, 3, 31, 7, 12], dtype=np.int64)
    write_pages, write_slots = np.array([0, 1, 2, 3, 1], dtype=np.int64), np.array([0, 1, 2, 3, 0], dtype=np.int64)
    cos, sin = rotary_tables(head_dim, 10000.0, capacity)
    gain_q = llama_ref.bf16(1.0 + 0.1 * rng.standard_normal(head_dim).astype(np.float32))
    gain_k = llama_ref.bf16(1.0 + 0.1 * rng.standard_normal(head_dim).astype(np.float32))
    norm_q, norm_k = which != "key without a gain", which != "query with a gain"
    use_gain_k = which == "both"
    d_k = torch.zeros((pages, page_size, kv_heads, head_dim), dtype=torch.bfloat16, device="cuda")
    d_v = torch.zeros_like(d_k)
    q_out = torch.empty((tokens, heads, head_dim), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    d_qkv, cos_d, sin_d = dev(qkv, torch.bfloat16), dev(cos, torch.bfloat16), dev(sin, torch.bfloat16)
    d_positions, d_pages, d_slots = dev(positions), dev(write_pages), dev(write_slots)
    d_gq, d_gk = dev(gain_q, torch.bfloat16), dev(gain_k, torch.bfloat16)
    code = ks.lib().singe_rotary_norm_cache_write_bf16(
        _stream(), q_out.data_ptr(), d_qkv.data_ptr(), qkv.shape[1], cos_d.data_ptr(), sin_d.data_ptr(),
        d_positions.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), d_pages.data_ptr(), d_slots.data_ptr(), 8, tokens,
        heads, kv_heads, head_dim, pages, page_size, capacity, int(norm_q), d_gq.data_ptr() if norm_q else None,
        int(norm_k), d_gk.data_ptr() if use_gain_k else None, eps, status.data_ptr())
    torch.cuda.synchronize()
    assert code == ks.OK and int(status.item()) == 0
    c, s = llama_ref.bf16(cos)[positions], llama_ref.bf16(sin)[positions]
    q = qkv[:, : heads * head_dim].reshape(tokens, heads, head_dim)
    k = qkv[:, heads * head_dim: (heads + kv_heads) * head_dim].reshape(tokens, kv_heads, head_dim)
    ones = np.ones(head_dim, dtype=np.float32)

    def normalised(x, gain):
        return llama_ref.rms_norm(x.reshape(-1, head_dim), gain, eps).reshape(x.shape)

    expect_q = llama_ref.rotate(normalised(q, gain_q) if norm_q else q, c, s)
    expect_k = llama_ref.rotate(normalised(k, gain_k if use_gain_k else ones) if norm_k else k, c, s)
    assert_close_bf16(host(q_out), expect_q, f"normalised + rotated queries ({which})")
    written = host(d_k)[write_pages, write_slots]
    assert_close_bf16(written, expect_k, f"normalised + rotated keys ({which})")
    if not norm_q:
        assert np.array_equal(host(q_out), expect_q)   # heads without a norm keep the exact rounding chain


@pytest.mark.parametrize("width", [4096, 50])
def test_embedding_and_argmax(width):
    rng = np.random.default_rng(width)
    vocab = 321
    table = workloads.normal_bf16(rng, (vocab, width))
    ids = np.array([0, 320, 7, -1, 400], dtype=np.int64)
    out = torch.empty((5, width), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    d_table, d_ids = dev(table, torch.bfloat16), dev(ids)
    assert ks.lib().singe_embedding_bf16(_stream(), out.data_ptr(), d_table.data_ptr(), d_ids.data_ptr(), 8, 5,
                                         width, vocab, status.data_ptr()) == ks.OK
    torch.cuda.synchronize()
    expect = np.stack([table[0], table[320], table[7], table[320], np.zeros(width, dtype=np.float32)])
    assert np.array_equal(host(out), expect) and int(status.item()) == 1   # id 400 is outside the table
    logits = workloads.normal_bf16(rng, (6, width))
    logits[2, 5] = logits[2, 9] = 50.0                                     # a tie: the lowest index wins
    best_value = torch.empty(6, device="cuda")
    best_index = torch.empty(6, dtype=torch.int64, device="cuda")
    d_logits = dev(logits, torch.bfloat16)
    assert ks.lib().singe_argmax_bf16(_stream(), best_value.data_ptr(), best_index.data_ptr(), d_logits.data_ptr(),
                                      width, 6, width, 1000) == ks.OK
    torch.cuda.synchronize()
    assert best_index.cpu().tolist() == (logits.argmax(axis=1) + 1000).tolist()
    assert best_index.cpu().tolist()[2] == 1005
    assert np.array_equal(best_value.cpu().numpy(), logits.max(axis=1))
