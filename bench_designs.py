"""`bench.py --design doderax`: prefill and decode throughput of the Doderax design at layer sizes that resemble a
real model's (random weights), beside the dense SwiGLU decoder of equal width, depth and parameter count, and every
kernel the design adds alone, with the fraction of its roofline, beside the like kernel of the dense decoder.

A kernel alone is launched 24 times inside one CUDA graph on rotating copies of its operands (together more than the
L2 holds); the graph is replayed five times and the median time per launch is taken from CUDA events.
"""

from __future__ import annotations

import statistics

PROMPT = 2048
BATCH = 8
PAGE = 16

# width, feed-forward, layers (three recurrent layers, then one with attention beside the recurrence), heads
DESIGN_SIZES = {
    "w2048": dict(width=2048, ff=8192, layers=12, heads=16, kv_heads=4, dim=128, window=1024, keep_first=4, vocab=65536),
    "w4096": dict(width=4096, ff=14336, layers=8, heads=32, kv_heads=8, dim=128, window=2048, keep_first=4, vocab=65536),
}


def doderax_config(s: dict) -> dict:
    delta = {"heads": s["heads"], "kv_heads": s["heads"], "dim": s["dim"], "vdim": s["dim"], "conv": 4,
             "decay_rank": 64, "gate_rank": 64}
    left = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
            "rot": {"dims": s["dim"] // 2, "base": 1000000.0}, "mask": {"size": s["window"], "keep_first": s["keep_first"]}}
    right = {"heads": s["heads"], "kv_heads": s["heads"] // 2, "dim": s["dim"], "vdim": s["dim"], "conv": 4}
    mlp = {"kind": "dense", "ff": s["ff"]}
    layers = [{"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp} if index % 4 == 3 else
              {"type": "channel_delta", "mixer": delta, "mlp": mlp} for index in range(s["layers"])]
    return {"architecture": "Doderax", "vocab": s["vocab"], "width": s["width"], "logit_scale": 1.0,
            "norm": {"eps": 1e-6}, "embedding": {"bigram": {"buckets": 65521, "mul_prev": 8191, "mul_cur": 131}},
            "layers": layers}


def dense_config(s: dict) -> dict:
    """The dense SwiGLU decoder of the same width, depth and heads; its three feed-forward matrices hold what the
    design's two hold."""
    inter = -(-(2 * s["ff"] // 3) // 128) * 128
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": s["width"],
            "intermediate_size": inter, "num_hidden_layers": s["layers"], "num_attention_heads": s["heads"],
            "num_key_value_heads": s["kv_heads"], "head_dim": s["dim"], "vocab_size": s["vocab"],
            "max_position_embeddings": 16384, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
            "tie_word_embeddings": False, "hidden_act": "silu"}


def run(args, peaks: dict) -> dict:
    import numpy as np
    import torch

    from libmir_b200 import CacheConfig, CudaConfig, Library, RuntimeConfig, SchedulerConfig, StepEntry, kernels
    from libmir_b200.sampling import RequestSampler

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    rng = np.random.default_rng(0)
    hbm, flops_peak = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    steps, warmup = args.steps, max(args.warmup, 3)
    bf16, f32, i32 = torch.bfloat16, torch.float32, torch.int32

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def model_numbers(config, vocab):
        pages = BATCH * (-(-(PROMPT + steps + warmup + 64) // PAGE)) + 64
        runtime = RuntimeConfig(kv_cache=CacheConfig(block_size=PAGE, block_count=pages),
                                scheduler=SchedulerConfig(max_batch_requests=BATCH, max_batch_tokens=8192,
                                                          prefill_chunk_tokens=4096),
                                cuda=CudaConfig(decode_graphs=True), dtype="bfloat16")
        model = Library(runtime).load_random(config, seed=0)
        for buffer in model.storage.buffers:
            buffer.normal_(0.0, 0.5)
        times = []
        tokens = rng.integers(0, vocab, size=PROMPT).tolist()
        for index in range(7):
            model.admit(f"p{index}")
            start, stop = events()
            torch.cuda.synchronize()
            start.record()
            result = model.step([StepEntry(f"p{index}", tokens, [PROMPT - 1])], [RequestSampler()])
            stop.record()
            torch.cuda.synchronize()
            result.tokens.cpu()
            model.release(f"p{index}")
            if index >= 2:
                times.append(start.elapsed_time(stop))
        prefill_ms = statistics.median(times)
        regions = []
        for _ in range(3):
            ids = []
            for index in range(BATCH):
                sequence = model.cache.admit(f"d{index}")
                model.cache.grow(sequence, PROMPT)
                model.cache.commit(sequence, PROMPT)
                sequence.last_token = 1                        # (the cache is synthetic: any token stands before)
                ids.append(f"d{index}")
            samplers = [RequestSampler() for _ in ids]
            entries = [StepEntry(i, [int(t)], [0]) for i, t in zip(ids, rng.integers(0, vocab, size=BATCH))]
            out = model.decode_many(entries, samplers, warmup)
            entries = [StepEntry(i, [int(t)], [0]) for i, t in zip(ids, out[-1].tolist())]
            torch.cuda.synchronize()
            start, stop = events()
            start.record()
            model.decode_many(entries, samplers, steps)
            stop.record()
            torch.cuda.synchronize()
            regions.append(start.elapsed_time(stop) / steps)
            for request_id in ids:
                model.release(request_id)
        decode_ms = statistics.median(regions)
        weight_bytes = model.decoder.weight_bytes_per_step()
        state_bytes = sum(t.numel() * t.element_size() // t.shape[0]
                          for held in model.storage.states.values()
                          for t in (held if isinstance(held, tuple) else (held,)))
        numbers = {"prefill_ms": round(prefill_ms, 3), "prefill_tokens_per_s": round(PROMPT * 1e3 / prefill_ms),
                   "decode_ms_per_step": round(decode_ms, 4), "decode_tokens_per_s": round(BATCH * 1e3 / decode_ms),
                   "weight_gb": round(weight_bytes / 1e9, 3), "state_mb_per_request": round(state_bytes / 1e6, 2)}
        model.unload()
        return numbers

    def timed(calls, work, peak, launches=24, repeats=5):
        for call in calls[:2]:
            call()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for index in range(launches):
                calls[index % len(calls)]()
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(repeats):
            start, stop = events()
            start.record()
            graph.replay()
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) * 1e3 / launches)
        us = statistics.median(times)
        return [round(us, 2), round(work / (us * 1e-6) / peak, 4)]

    def copies(make, bytes_each):
        return [make() for _ in range(max(2, min(24, -(-(300 << 20) // max(bytes_each, 1)))))]

    def kernel_table(s):
        heads, kv_heads, dim, width, ff = s["heads"], s["kv_heads"], s["dim"], s["width"], s["ff"]
        table = {}
        rand = lambda *shape, dtype=bf16, scale=1.0: (torch.randn(*shape, device=device, dtype=f32) * scale).to(dtype)
        for label, rows, portion in ((f"prefill_{PROMPT}", 1, PROMPT), (f"decode_b{BATCH}", BATCH, 1)):
            tokens = rows * portion
            starts = torch.arange(0, tokens + 1, portion, dtype=i32, device=device)
            row_of = torch.arange(tokens, dtype=i32, device=device) // portion
            positions = torch.full((tokens,), PROMPT, dtype=i32, device=device)
            # the recurrence: state [slots, H, V, D] read and written once per step; 4 D V multiply-adds per token and head
            for per_channel, name in ((True, "delta_rule_channel"), (False, "delta_rule_head")):
                decay_width = heads * dim if per_channel else heads
                packs = copies(lambda: (torch.zeros(rows, heads, dim, dim, device=device, dtype=f32),
                                        rand(tokens, 3 * heads * dim, dtype=f32, scale=0.1)),
                               rows * heads * dim * dim * 4)
                beta = torch.rand(tokens, heads, device=device, dtype=f32)
                decay = torch.rand(tokens, decay_width, device=device, dtype=f32) * 0.5 + 0.5
                out = torch.empty(tokens, heads * dim, device=device, dtype=f32)
                slots = torch.arange(rows, dtype=i32, device=device)
                calls = [lambda p=p: kernels.delta_rule_scan(p[1], beta, decay, p[0], starts, slots, positions, out, heads,
                                                             heads, dim, dim) for p in packs]
                state_bytes = rows * heads * dim * dim * 4 * 2 + tokens * (3 * heads * dim + decay_width + heads * dim) * 4
                if portion == 1:
                    table[f"{label}_{name}"] = timed(calls, state_bytes, hbm)
                else:   # a prompt: the state stays in registers; the work is 32-bit multiply-adds, no tensor cores
                    table[f"{label}_{name}"] = timed(calls, 8.0 * tokens * heads * dim * dim, flops_peak) + ["of the bf16 tensor peak; the kernel is 32-bit FMA, one token after the other"]
                # the parallel pass before it: convolution, unit vectors, gates
                raw = rand(tokens, 3 * heads * dim + 64)
                conv_w = rand(3 * heads * dim, 4)
                conv_tail = torch.zeros(rows, 3, 3 * heads * dim, device=device, dtype=f32)
                beta_raw = rand(tokens, heads)
                decay_raw = rand(tokens, decay_width, dtype=f32 if per_channel else bf16)
                bias, a_log = rand(decay_width, dtype=f32), rand(heads, dtype=f32, scale=0.3)
                prepared = [torch.empty(tokens, 3 * heads * dim, device=device, dtype=f32) for _ in range(4)]
                decay_out = torch.empty(tokens, decay_width, device=device, dtype=f32)
                calls = [lambda o=o: kernels.delta_rule_prepare(raw[:, :3 * heads * dim], conv_w, conv_tail, beta_raw, decay_raw,
                                                                bias, a_log, row_of, starts, slots, positions, o, beta,
                                                                decay_out, heads, heads, dim, dim) for o in prepared]
                moved = tokens * (3 * heads * dim * 6 + decay_width * 8)
                table[f"{label}_{name}_prepare"] = timed(calls, moved, hbm)
            channels = 3 * heads * dim
            packs = copies(lambda: rand(tokens, channels + 64), tokens * channels * 2)
            weight = rand(channels, 4)
            tail = torch.zeros(rows, 3, channels, device=device, dtype=f32)
            out = torch.empty(tokens, channels, device=device, dtype=f32)
            slots = torch.arange(rows, dtype=i32, device=device)
            calls = [lambda p=p: kernels.short_conv_silu(p[:, :channels], weight, tail, row_of, starts, slots, positions, out)
                     for p in packs]
            table[f"{label}_short_conv_silu"] = timed(calls, tokens * channels * 6 + rows * 3 * channels * 8, hbm)
            packs = copies(lambda: (rand(tokens, heads * dim, dtype=f32), rand(tokens, heads * dim)), tokens * heads * dim * 6)
            norm_weight = rand(dim, dtype=f32)
            out16 = torch.empty(tokens, heads * dim, device=device, dtype=bf16)
            calls = [lambda p=p: kernels.gated_head_norm(p[0], p[1], norm_weight, out16, heads, dim, 1e-6, True) for p in packs]
            table[f"{label}_gated_head_norm"] = timed(calls, tokens * heads * dim * 8, hbm)
            packs = copies(lambda: (rand(tokens, width, dtype=f32), rand(tokens, width, dtype=f32), rand(tokens, width, dtype=f32)),
                           tokens * width * 12)
            w_a, w_b = rand(width, dtype=f32), rand(width, dtype=f32)
            calls = [lambda p=p: kernels.add_normed_branches([p[0], p[1]], [w_a, w_b], p[2], 1e-6, 0.5) for p in packs]
            table[f"{label}_add_normed_branches"] = timed(calls, tokens * width * 16, hbm)
            packs = copies(lambda: rand(tokens, ff), tokens * ff * 2)
            calls = [lambda p=p: kernels.gelu_tanh(p) for p in packs]
            table[f"{label}_gelu_tanh"] = timed(calls, tokens * ff * 4, hbm)
            # the dense decoder's elementwise kernels for comparison
            packs = copies(lambda: rand(tokens, width, dtype=f32), tokens * width * 4)
            out_w = torch.empty(tokens, width, device=device, dtype=bf16)
            calls = [lambda p=p: kernels.rms_norm(p, w_a, 1e-6, out_w) for p in packs]
            table[f"{label}_dense_rms_norm"] = timed(calls, tokens * width * 6, hbm)
            inter = ff * 2 // 3 // 128 * 128
            packs = copies(lambda: rand(tokens, 2 * inter), tokens * inter * 4)
            out_i = torch.empty(tokens, inter, device=device, dtype=bf16)
            calls = [lambda p=p: kernels.silu_mul(p, out_i) for p in packs]
            table[f"{label}_dense_silu_mul"] = timed(calls, tokens * inter * 6, hbm)
            # attention: a window with kept first keys (the tile kernel) beside the dense decoder's kernels, same sizes
            context = PROMPT if portion > 1 else PROMPT + 1
            pages_per_row = -(-(context + PAGE) // PAGE)
            cache_rows = rows * pages_per_row * PAGE
            layers = max(2, min(24, -(-(300 << 20) // (cache_rows * kv_heads * dim * 4))))
            k_cache = [rand(cache_rows, kv_heads, dim, scale=0.5) for _ in range(layers)]
            v_cache = [rand(cache_rows, kv_heads, dim, scale=0.5) for _ in range(layers)]
            block_table = torch.arange(rows * pages_per_row, dtype=i32, device=device).view(rows, pages_per_row).contiguous()
            contexts = torch.full((rows,), context, dtype=i32, device=device)
            q_positions = torch.full((tokens,), context - 1, dtype=i32, device=device)
            qkv = rand(tokens, (heads + 2 * kv_heads) * dim, scale=0.3)
            mixed = torch.empty(tokens, heads * dim, device=device, dtype=bf16)
            window = s["window"]
            scale = dim ** -0.5
            calls = [lambda k=k, v=v: kernels.prefill_attention(qkv, mixed, k, v, block_table, starts, contexts, PAGE, heads,
                                                                 kv_heads, dim, scale, window,
                                                                 keep_first=s["keep_first"]) for k, v in zip(k_cache, v_cache)]
            if portion > 1:
                visible = sum(min(p + 1, window) for p in range(PROMPT))
                flops = 4.0 * visible * dim * heads
                table[f"{label}_attention_window_kept"] = timed(calls, flops, flops_peak)
                calls = [lambda k=k, v=v: kernels.prefill_attention(qkv, mixed, k, v, block_table, starts, contexts, PAGE,
                                                                     heads, kv_heads, dim, scale, window) for k, v in zip(k_cache, v_cache)]
                table[f"{label}_dense_attention_window"] = timed(calls, flops, flops_peak)
                calls = [lambda k=k, v=v: kernels.prefill_attention(qkv, mixed, k, v, block_table, starts, contexts, PAGE,
                                                                     heads, kv_heads, dim, scale, None) for k, v in zip(k_cache, v_cache)]
                table[f"{label}_dense_attention_full"] = timed(calls, 4.0 * (PROMPT * (PROMPT + 1) / 2) * dim * heads, flops_peak)
            else:
                key_bytes = rows * min(window, context) * kv_heads * dim * 2 * 2
                partition, count, floats = kernels.decode_attention_kept_plan(rows, heads, dim, context)
                scratch = torch.empty(max(floats, 1), device=device, dtype=f32)
                numbering = torch.empty(rows, device=device, dtype=i32)
                calls = [lambda k=k, v=v: kernels.decode_attention(qkv, mixed, k, v, block_table, q_positions, PAGE, heads,
                                                                    kv_heads, dim, scale, window, partition, count, scratch,
                                                                    keep_first=s["keep_first"], numbering=numbering)
                         for k, v in zip(k_cache, v_cache)]
                table[f"{label}_attention_window_kept"] = timed(calls, key_bytes, hbm)
                for span, name in ((window, "dense_attention_window"), (None, "dense_attention_full")):
                    partition, count, floats = kernels.decode_attention_plan(rows, heads, kv_heads, dim, PAGE, context)
                    scratch = torch.empty(max(floats, 1), device=device, dtype=f32)
                    calls = [lambda k=k, v=v: kernels.decode_attention(qkv, mixed, k, v, block_table, q_positions, PAGE, heads,
                                                                        kv_heads, dim, scale, span, partition, count,
                                                                        scratch if floats else None)
                             for k, v in zip(k_cache, v_cache)]
                    read = rows * (min(span, context) if span else context) * kv_heads * dim * 2 * 2
                    table[f"{label}_{name}"] = timed(calls, read, hbm)
        return table

    chosen = [name for name in DESIGN_SIZES if args.design_sizes in ("all", name)]
    report = {}
    for name in chosen:
        s = DESIGN_SIZES[name]
        entry = {"sizes": s}
        if not args.skip_points:
            entry["kernels_us_and_fraction_of_roofline"] = kernel_table(s)
        entry["doderax"] = model_numbers(doderax_config(s), s["vocab"])
        entry["dense_swiglu"] = model_numbers(dense_config(s), s["vocab"])
        report[name] = entry
    return report
