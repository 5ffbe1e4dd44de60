"""Secondary figures reported beside the headline decode number: the other kernels of the hot path on their
own benchmark configurations (config 3 GEMM shapes, config 4 prefill and cache write), each as achieved
throughput and as a fraction of the measured roofline.  Inputs are seeded synthetic tensors created on the
device; every kernel is timed with CUDA events around a CUDA graph of repeated launches.
"""
from __future__ import annotations

import numpy as np
import torch

from singe_b200 import ops, workloads


def graph_seconds(fn, reps: int = 10, rounds: int = 3) -> float:
    """Average duration of one call of ``fn`` inside a CUDA graph of ``reps`` launches (best of ``rounds``)."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(reps):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(rounds):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            graph.replay()
            end.record(stream)
            torch.cuda.synchronize()
            best = min(best, begin.elapsed_time(end) * 1e-3 / reps)
    return best


L2_BYTES = 126 << 20


def rotating(make_call, set_bytes: int, minimum: int = 4):
    """``make_call(i)`` builds the call on operand set i.  Returns one function that walks through enough distinct
    sets (at least ``minimum``, and more than twice the L2's capacity in total) so that no launch finds the operands of
    an earlier one in the 126 MB L2: what is timed is then HBM traffic, not cache hits."""
    sets = max(minimum, -(-2 * L2_BYTES // max(set_bytes, 1)) + 1)
    calls = [make_call(i) for i in range(sets)]
    state = {"next": 0}

    def call():
        calls[state["next"] % sets]()
        state["next"] += 1

    return call, sets


def gemm_figures(peaks) -> dict:
    """Config 3.  The weight-streaming shapes (M <= 128) are HBM-bound: each is timed over rotating weight matrices
    (see ``rotating``) and, for comparison, also the old way on one matrix that partly stays in L2."""
    out = {}
    generator = torch.Generator(device="cuda").manual_seed(2)
    for n, k in workloads.GEMM_SHAPES:
        weight_bytes = 2 * n * k
        sets = max(4, -(-2 * L2_BYTES // weight_bytes) + 1)
        weights = [(torch.randn((n, k), generator=generator, device="cuda") * 0.02).to(torch.bfloat16)
                   for _ in range(sets)]
        for m in workloads.GEMM_ROWS:
            x = torch.randn((m, k), generator=generator, device="cuda").to(torch.bfloat16)
            y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
            flops = 2.0 * m * n * k
            moved = 2.0 * (m * k + n * k + m * n)
            if m == 4096:
                seconds = graph_seconds(lambda: ops.linear(x, weights[0], y), reps=4)
                entry = {"us": round(seconds * 1e6, 2), "tflops": round(flops / seconds / 1e12, 1),
                         "frac_of_bf16_peak": round(flops / seconds / 1e12 / peaks["bf16_tflops"], 4)}
            else:
                call, used = rotating(lambda i: (lambda: ops.linear(x, weights[i], y)), weight_bytes)
                reps = 2 * used
                seconds = graph_seconds(call, reps=reps)
                resident = graph_seconds(lambda: ops.linear(x, weights[0], y), reps=10)
                entry = {"us": round(seconds * 1e6, 2), "gbs": round(moved / seconds / 1e9, 1),
                         "frac_of_hbm_peak": round(moved / seconds / 1e9 / peaks["hbm_gbs"], 4),
                         "l2": f"rotated, {used} weight matrices",
                         "same_matrix_every_launch": {"us": round(resident * 1e6, 2),
                                                      "gbs": round(moved / resident / 1e9, 1),
                                                      "note": "partly L2-resident: not an HBM figure"}}
            out[f"M{m}_N{n}_K{k}"] = entry
        del weights
        torch.cuda.empty_cache()
    return out


def cache_write_figures(peaks) -> dict:
    case = workloads.prefill_case()
    total = case.total_tokens
    shape = (case.pages, case.page_size, case.kv_heads, case.head_dim)
    key_cache = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    value_cache = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    pages = torch.from_numpy(case.write_pages).cuda()
    slots = torch.from_numpy(case.write_slots).cuda()
    moved = 4.0 * total * case.kv_heads * case.head_dim * 2  # K and V rows read once and written once

    def make(i):
        # every set has its own source rows and its own cache: nothing a launch touches is left in L2 by another
        keys = torch.randn((total, case.kv_heads, case.head_dim), device="cuda").to(torch.bfloat16)
        values = torch.randn((total, case.kv_heads, case.head_dim), device="cuda").to(torch.bfloat16)
        k_cache, v_cache = (key_cache, value_cache) if i == 0 else (torch.zeros_like(key_cache),
                                                                    torch.zeros_like(value_cache))
        return lambda: ops.kv_cache_write(k_cache, v_cache, keys, values, pages, slots)

    call, used = rotating(make, int(moved))
    seconds = graph_seconds(call, reps=2 * used)
    return {"us": round(seconds * 1e6, 2), "gbs": round(moved / seconds / 1e9, 1),
            "frac_of_hbm_peak": round(moved / seconds / 1e9 / peaks["hbm_gbs"], 4), "bytes": int(moved),
            "l2": f"rotated, {used} source/destination sets"}


def prefill_figures(peaks) -> dict:
    case = workloads.prefill_case()
    total = case.total_tokens
    generator = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn((total, case.heads, case.head_dim), generator=generator, device="cuda").to(torch.bfloat16)
    k = torch.randn((total, case.kv_heads, case.head_dim), generator=generator, device="cuda").to(torch.bfloat16)
    v = torch.randn((total, case.kv_heads, case.head_dim), generator=generator, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    lse = torch.empty((total, case.heads), dtype=torch.float32, device="cuda")
    lens = torch.from_numpy(case.lens).cuda()
    offsets = torch.from_numpy(case.offsets).cuda()
    shape = (case.pages, case.page_size, case.kv_heads, case.head_dim)
    key_cache = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    value_cache = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    pages = torch.from_numpy(case.write_pages).cuda()
    slots = torch.from_numpy(case.write_slots).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    config = ops.RaggedKvPrefillAttentionConfig(len(case.lens), total, total, case.heads, case.kv_heads,
                                                case.head_dim, True, case.scale)
    seconds = graph_seconds(
        lambda: ops.ragged_kv_prefill_attention(out, lse, q, k, v, lens, lens, offsets, config,
                                                cache_write=(key_cache, value_cache, pages, slots, status)),
        reps=3)
    flops = case.causal_flops()
    figures = {"us": round(seconds * 1e6, 1), "tflops": round(flops / seconds / 1e12, 1),
               "frac_of_bf16_peak": round(flops / seconds / 1e12 / peaks["bf16_tflops"], 4),
               "causal_gflop": round(flops / 1e9, 1), "includes": "slot-mapped KV-cache write of all 15360 tokens"}
    # The same attention read back out of the cache the call above filled: K/V tiles gathered page by page.
    table = torch.from_numpy(case.block_table.view(np.int32)).cuda()
    paged_out = torch.empty_like(q)
    paged_lse = torch.empty_like(lse)
    paged = ops.PagedKvPrefillAttentionConfig(len(case.lens), total, case.heads, case.kv_heads, case.head_dim,
                                              case.page_size, case.pages, case.block_table.shape[1], True, case.scale)
    seconds = graph_seconds(
        lambda: ops.paged_kv_prefill_attention(paged_out, paged_lse, q, key_cache, value_cache, lens, lens, offsets,
                                               table, paged),
        reps=3)
    torch.cuda.synchronize()
    if not torch.allclose(paged_out.float(), out.float(), atol=2e-2, rtol=1e-2):
        raise RuntimeError("paged prefill differs from ragged prefill over the same keys and values")
    figures["paged"] = {"us": round(seconds * 1e6, 1), "tflops": round(flops / seconds / 1e12, 1),
                        "frac_of_bf16_peak": round(flops / seconds / 1e12 / peaks["bf16_tflops"], 4),
                        "bit_identical_to_ragged": bool(torch.equal(paged_out, out)),
                        "reads": "K/V from the 16-token cache pages through the block table"}
    return figures


def paged_attention_call():
    """Config 2 through the Tensor-surface entry point (FlashInfer-style paging, base-2 LSE, status word): returns
    (call, case, status) with every buffer resident on the device."""
    import numpy as np

    from singe_b200 import kernel_sys as ks

    case = workloads.paged_decode_case()
    generator = torch.Generator(device="cuda").manual_seed(1)
    shape = (case.physical_blocks, case.block_size, case.kv_heads, case.head_dim)
    key_cache = torch.randn(shape, generator=generator, device="cuda").to(torch.bfloat16)
    value_cache = torch.randn(shape, generator=generator, device="cuda").to(torch.bfloat16)
    query = torch.randn((case.batch, case.heads, case.head_dim), generator=generator, device="cuda").to(torch.bfloat16)
    blocks = (case.lens.astype(np.int64) + case.block_size - 1) // case.block_size
    page_offsets = np.concatenate([[0], np.cumsum(blocks)]).astype(np.int64)
    pages = np.concatenate([case.block_table[b, : blocks[b]] for b in range(case.batch)]).astype(np.int64)
    last = (case.lens.astype(np.int64) - (blocks - 1) * case.block_size).astype(np.int64)
    query_offsets = np.arange(case.batch + 1, dtype=np.int64)
    d = lambda a: torch.from_numpy(a).cuda()
    d_qo, d_po, d_pages, d_last = d(query_offsets), d(page_offsets), d(pages), d(last)
    out = torch.empty_like(query)
    lse = torch.empty((case.batch, case.heads), dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    fn = ks.lib().singe_paged_attention_bf16

    def call():
        stream = int(torch.cuda.current_stream().cuda_stream)
        code = fn(stream, out.data_ptr(), lse.data_ptr(), query.data_ptr(), key_cache.data_ptr(),
                  value_cache.data_ptr(), d_qo.data_ptr(), d_po.data_ptr(), d_pages.data_ptr(), d_last.data_ptr(), 8,
                  case.batch, case.heads, case.kv_heads, case.head_dim, case.block_size, case.physical_blocks,
                  case.batch, pages.size, case.scale, 1, 0, status.data_ptr())
        if code != ks.OK:
            raise RuntimeError(f"paged_attention: status {code}")

    return call, case, status


def paged_attention_figures(peaks) -> dict:
    call, case, status = paged_attention_call()
    seconds = graph_seconds(call)
    moved = float(case.algorithmic_bytes())
    return {"us": round(seconds * 1e6, 2), "gbs": round(moved / seconds / 1e9, 1),
            "frac_of_hbm_peak": round(moved / seconds / 1e9 / peaks["hbm_gbs"], 4),
            "status_word": int(status.item())}


def run_all(peaks) -> dict:
    result = {}
    for name, fn in (("kv_cache_write_config4", cache_write_figures), ("gemm_config3", gemm_figures),
                     ("prefill_config4", prefill_figures), ("paged_attention_config2", paged_attention_figures)):
        try:
            result[name] = fn(peaks)
        except Exception as error:
            result[name] = {"error": repr(error)}
    if ops.take_device_error() != 0:
        result["device_error"] = "a bounded wait ran out"
    return result
