#!/usr/bin/env python3
"""Decode and prefill throughput of the LFM2-1.2B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B]

Prints ONE JSON line.  ``value`` is decoded tokens a second at the given batch
(device time over exactly K decode steps, CUDA events); ``e2e`` is the same
through the Python entry point, with token ids coming from and going to the
host every step; ``prefill`` times one whole prompt of 2,048 tokens; ``roofline``
relates the decode step to the memory bandwidth; ``points`` holds batch 1 and 64.  The region of K decode steps is timed five times
back to back; ``value`` and ``e2e`` are the median region's, with the spread
((slowest - fastest) / median) beside them.
The model has random bfloat16 weights and uniform-random token ids (there is
neither a checkpoint nor a dataset here).  Decode steps read 2.3 GB of
weights each, far more than the L2 holds, so no flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the benchmark configuration: layer sizes of the LFM2-1.2B shape
LFM2_1P2B = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2", hidden_size=2048, num_hidden_layers=16,
    num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=65536, intermediate_size=12288,
    block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256, conv_L_cache=3,
    conv_bias=False, full_attn_idxs=[2, 5, 8, 10, 12, 14], rope_theta=1000000.0, norm_eps=1e-5, tie_embedding=True,
    max_position_embeddings=4096,
)
SEED, PROMPT_LEN, CONTEXT = 2, 2048, 4096
REPEATS = 5             # regions of K decode steps timed back to back; the median is reported


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "MisterTK/gibbs is a Rust crate with Apple Metal kernels: pip cannot install it "
                      "(no setup.py or pyproject.toml), there is no cargo/rustc here, and it has no CUDA path"}))
    return 0


def potivik_shape(size: str) -> dict:
    """Layer sizes that resemble a real model's, for the Potivik design: state-space and latent-attention
    layers in turn, a dense gated unit behind the former and routed experts behind the latter."""
    if size == "1k":
        d, vocab, side = 1024, 32768, 128
        ssm = {"heads": 32, "vdim": 64, "state": 64, "groups": 4, "conv": 4, "norm_groups": 4}
        att = {"heads": 8, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 256, "scale": 96 ** -0.5,
               "mask": {"size": 512}, "rot": {"base": 500000.0, "dims": 32}}
        dense = {"kind": "dense", "ff": 4096, "limit": 7.0}
        moe = {"kind": "moe", "router": {"experts": 16, "top": 2}, "expert": {"ff": 512, "limit": 7.0},
               "shared": {"ff": 1024, "limit": 7.0}}
    else:
        d, vocab, side = 2048, 65536, 256
        ssm = {"heads": 64, "vdim": 64, "state": 128, "groups": 8, "conv": 4, "norm_groups": 8}
        att = {"heads": 16, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5,
               "mask": {"size": 1024}, "rot": {"base": 500000.0, "dims": 64}}
        dense = {"kind": "dense", "ff": 8192, "limit": 7.0}
        moe = {"kind": "moe", "router": {"experts": 32, "top": 4}, "expert": {"ff": 1024, "limit": 7.0},
               "shared": {"ff": 2048, "limit": 7.0}}
    layers = []
    for i in range(8):
        layers.append({"type": "mamba2", "mixer": ssm, "mlp": dense} if i % 2 == 0 else
                      {"type": "latent_attention", "mixer": att, "mlp": moe})
    return {"architecture": "Potivik", "vocab": vocab, "width": d, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
            "token_side": {"dim": side}, "layers": layers}


def petelix_shape(size: str) -> dict:
    """Layer sizes that resemble a real model's, for the Petelix design: attention layers with routed experts,
    every second layer reading the keys and values of the layer before it."""
    if size == "1k":
        d, vocab = 1024, 32768
        att = {"heads": 16, "kv_heads": 4, "dim": 64, "vdim": 32, "scale": 0.125, "softcap": 30.0, "mask": {"size": 512},
               "rot": {"base": 500000.0, "dims": 32}}
        moe = {"kind": "moe", "router": {"experts": 14, "identity": 2, "top": 2, "groups": {"count": 4, "keep": 2}},
               "expert": {"ff": 1024}}
    else:
        d, vocab = 2048, 65536
        att = {"heads": 32, "kv_heads": 8, "dim": 64, "vdim": 64, "scale": 0.125, "softcap": 30.0, "mask": {"size": 1024},
               "rot": {"base": 500000.0, "dims": 32}}
        moe = {"kind": "moe", "router": {"experts": 30, "identity": 2, "top": 4, "groups": {"count": 4, "keep": 2}},
               "expert": {"ff": 1024}}
    layers = [{"type": "attention", "mixer": dict(att, **({"kv_from": i - 1} if i % 2 else {})), "mlp": moe} for i in range(8)]
    return {"architecture": "Petelix", "vocab": vocab, "width": d, "norm": {"eps": 1e-6}, "embedding": {"scale": 8.0},
            "layers": layers}


def sisadra_shape(size: str) -> dict:
    """Layer sizes that resemble a real model's, for the Sisadra design: delta-rule layers in turn with
    differential attention in blocks and latent attention, a dense feed-forward behind each."""
    if size == "1k":
        d, vocab = 1024, 32768
        rule = {"heads": 16, "kv_heads": 8, "dim": 64, "vdim": 64, "conv": 4, "decay_rank": 64, "gate_rank": 64}
        att = {"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 128, "scale": 0.125, "diff": 0.3, "mask": {"size": 512},
               "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
        lat = {"heads": 8, "dim": 64, "vdim": 64, "kv_rank": 256, "scale": 0.125}
    else:
        d, vocab = 2048, 65536
        rule = {"heads": 16, "kv_heads": 8, "dim": 128, "vdim": 128, "conv": 4, "decay_rank": 128, "gate_rank": 128}
        att = {"heads": 16, "kv_heads": 4, "dim": 64, "vdim": 128, "scale": 0.125, "diff": 0.3, "mask": {"size": 1024},
               "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
        lat = {"heads": 16, "dim": 128, "vdim": 128, "kv_rank": 512, "scale": 128 ** -0.5}
    mlp = {"kind": "dense", "ff": 4 * d}
    kinds = ["channel_delta", "attention", "channel_delta", "latent_attention"] * 2
    mixers = {"channel_delta": rule, "attention": att, "latent_attention": lat}
    return {"architecture": "Sisadra", "vocab": vocab, "width": d, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
            "embedding": {"scale": 8.0, "bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 999983}},
            "layers": [{"type": k, "mixer": mixers[k], "mlp": mlp} for k in kinds]}


def selivik_shape(size: str) -> dict:
    """Layer sizes that resemble a real model's, for the Selivik design: latent-attention layers in turn with
    windowed attention layers that keep a sequence's first positions; a dense gated unit behind the first layer
    of every four, routed experts behind the others."""
    if size == "1k":
        d, vocab = 1024, 32768
        att = {"heads": 16, "kv_heads": 4, "dim": 64, "vdim": 64, "scale": 0.125, "softcap": 30.0,
               "mask": {"size": 512, "keep_first": 64}, "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0}}}
        lat = {"heads": 8, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 256, "q_rank": 384, "scale": 96 ** -0.5,
               "rot": {"base": 10000.0, "dims": 32}}
        dense = {"kind": "dense", "ff": 4096}
        moe = {"kind": "moe", "router": {"experts": 16, "top": 2}, "expert": {"ff": 1024}}
    else:
        d, vocab = 2048, 65536
        att = {"heads": 32, "kv_heads": 8, "dim": 64, "vdim": 64, "scale": 0.125, "softcap": 30.0,
               "mask": {"size": 1024, "keep_first": 128}, "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0}}}
        lat = {"heads": 16, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "q_rank": 768, "scale": 192 ** -0.5,
               "rot": {"base": 10000.0, "dims": 64}}
        dense = {"kind": "dense", "ff": 8192}
        moe = {"kind": "moe", "router": {"experts": 32, "top": 4}, "expert": {"ff": 1024}}
    four = [("latent_attention", lat, dense), ("attention", att, moe), ("latent_attention", lat, moe), ("attention", att, moe)]
    return {"architecture": "Selivik", "vocab": vocab, "width": d, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "embedding": {"scale": 8.0}, "layers": [{"type": k, "mixer": m, "mlp": f} for k, m, f in four * 2]}


def potivik_workload(a):
    """Prompt and decode throughput of the Potivik design at two sizes (random weights), beside an LFM2
    model of equal width, depth and feed-forward width, with the time per kind of operation of one
    prompt step and one decode step (the walker's timing mode).  One JSON line per model and size.
    'petelix': the same for the Petelix design, beside an LFM2 model whose layers are all attention layers
    and whose feed-forward is as wide as the experts a token uses.  'sisadra': the same for the Sisadra design,
    beside an LFM2 model and a Potivik model (state-space and latent-attention layers in turn) of equal width,
    depth and feed-forward width.  'selivik': the Selivik design beside an LFM2 model, a Petelix model (windowed
    attention with a sink and routed experts) and a Potivik model (latent attention with a rotated part) of equal
    width and depth."""
    import torch
    from gibbs_b200 import Engine, Lfm2Config, parse_config, random_model
    from gibbs_b200.engine import benchmark as B
    prompt, batch, ctx = 2048, 8, 1024
    for size in (a.size.split(",") if a.size else ["1k", "2k"]):
        if a.workload == "petelix":
            pot = petelix_shape(size)
            d, m, r = pot["width"], pot["layers"][0]["mixer"], pot["layers"][0]["mlp"]["router"]
            twin = dict(LFM2_1P2B, hidden_size=d, num_hidden_layers=8, num_attention_heads=m["heads"],
                        num_key_value_heads=m["kv_heads"], head_dim=m["dim"], vocab_size=pot["vocab"],
                        intermediate_size=r["top"] * pot["layers"][0]["mlp"]["expert"]["ff"], block_auto_adjust_ff_dim=False,
                        full_attn_idxs=list(range(8)), max_position_embeddings=4096)
        elif a.workload == "sisadra":
            pot = sisadra_shape(size)
            d = pot["width"]
            twin = dict(LFM2_1P2B, hidden_size=d, num_hidden_layers=8, num_attention_heads=d // 64, num_key_value_heads=d // 256,
                        head_dim=64, vocab_size=pot["vocab"], intermediate_size=4 * d, block_auto_adjust_ff_dim=False,
                        full_attn_idxs=[1, 3, 5, 7], max_position_embeddings=4096)
        elif a.workload == "selivik":
            pot = selivik_shape(size)
            d = pot["width"]
            twin = dict(LFM2_1P2B, hidden_size=d, num_hidden_layers=8, num_attention_heads=d // 64, num_key_value_heads=d // 256,
                        head_dim=64, vocab_size=pot["vocab"], intermediate_size=4 * d, block_auto_adjust_ff_dim=False,
                        full_attn_idxs=[1, 3, 5, 7], max_position_embeddings=4096)
        else:
            pot = potivik_shape(size)
            d = pot["width"]
            twin = dict(LFM2_1P2B, hidden_size=d, num_hidden_layers=8, num_attention_heads=d // 64, num_key_value_heads=d // 256,
                        head_dim=64, vocab_size=pot["vocab"], intermediate_size=4 * d, block_auto_adjust_ff_dim=False,
                        full_attn_idxs=[1, 3, 5, 7], max_position_embeddings=4096)
        models = [(pot["architecture"], parse_config(pot)), ("LFM2 of equal size", Lfm2Config.from_dict(twin))]
        if a.workload == "sisadra":
            models.append(("Potivik of equal size", parse_config(potivik_shape(size))))
        if a.workload == "selivik":
            models.append(("Petelix of equal size", parse_config(petelix_shape(size))))
            models.append(("Potivik of equal size", parse_config(potivik_shape(size))))
        for name, conf in models:
            model = random_model(conf, SEED, dtype="bfloat16", device="cuda:0", stored_dtype=torch.bfloat16)
            eng = Engine(model, n_pages=(batch + 1) * (4096 // 16), page_size=16, max_requests=batch, max_step_tokens=prompt,
                         max_context=4096)
            pre = B.measure_prefill(eng, prompt, warmup=3, runs=5, seed=SEED)
            dec = B.measure_decode(eng, batch, ctx, a.steps, max(a.warmup, 3), seed=SEED)
            line = {"model": name, "width": d, "layers": 8, "prompt_tokens": prompt, "prefill_ms": round(pre["ms"], 3),
                    "prefill_tok_s": round(pre["value"], 1), "decode_batch": batch, "decode_context": dec["context"],
                    "decode_ms_per_step": round(dec["ms_per_step"], 4), "decode_tok_s": round(dec["tok_s"], 1),
                    "decode_gbs": round(dec["gbs"], 1), "launches_per_decode_step": dec["launches"] // max(a.steps, 1),
                    "prefill_kind_ms": B.prefill_kind_times(eng, prompt, seed=SEED),
                    "decode_kind_us": B.decode_kind_times(eng, batch, ctx, seed=SEED),
                    "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), uniform-random token ids"}
            print(json.dumps(line), flush=True)
            del eng, model
            torch.cuda.empty_cache()
    return 0


def other_workload(a):
    """The two other workloads this project's configurations name: mixed serving at the
    LFM2-700M shape, and a long context at the LFM2-2.6B shape."""
    import torch
    from gibbs_b200 import Generator, Lfm2Config, random_model
    from gibbs_b200.engine import benchmark as B
    base = dict(LFM2_1P2B)
    if a.workload == "serve700m":
        base.update(hidden_size=1536, num_attention_heads=24, intermediate_size=10240, max_position_embeddings=4096)
        cfg = Lfm2Config.from_dict(base)
        model = random_model(cfg, 3, dtype="bfloat16", device="cuda:0")
        gen = Generator(model, ctx=2048 + 256 + 16, page_size=16, max_running=64, max_batch_tokens=512, seed=3)
        B.measure_serving(gen, n_requests=64, min_len=16, max_len=2048, new_tokens=256, temperature=0.8, seed=1)  # warm-up
        res = B.measure_serving(gen, n_requests=64, min_len=16, max_len=2048, new_tokens=256, temperature=0.8, seed=3)
        res["workload"] = "LFM2-700M shape: 64 requests, prompts U[16, 2048], portions of 512 beside decode, 256 new tokens, T=0.8"
    elif a.workload == "sweep":
        # the benchmark's shape at other batch sizes, contexts and prompt lengths: one JSON line per point
        from gibbs_b200 import Engine
        base.update(max_position_embeddings=32768 + 256)
        model = random_model(Lfm2Config.from_dict(base), SEED, dtype="bfloat16", device="cuda:0")
        pk = B.load_peaks(os.path.join(ROOT, "MEASURED_PEAKS.json"))
        hbm, tensor = pk["hbm_gbs"], pk["bf16_tflops"]
        for ctx in (512, 2048, 8192, 32768):
            for batch in (1, 8, 64):
                if batch * ctx > 600_000:
                    continue
                eng = Engine(model, n_pages=batch * (ctx // 16 + 8), page_size=16, max_requests=batch,
                             max_step_tokens=2048, max_context=ctx + 128)
                d = B.measure_decode(eng, batch, ctx, 32, 4, seed=SEED)
                print(json.dumps({"decode_batch": batch, "context": d["context"], "ms_per_step": round(d["ms_per_step"], 4),
                                  "tok_s": round(d["tok_s"], 1), "gbs": round(d["gbs"], 1),
                                  "hbm_frac": round(d["gbs"] / hbm, 3)}), flush=True)
                del eng
                torch.cuda.empty_cache()
        for n in (128, 512, 2048, 8192):
            eng = Engine(model, n_pages=n // 16 + 8, page_size=16, max_requests=1, max_step_tokens=n, max_context=n + 16)
            pre = B.measure_prefill(eng, n, warmup=2, runs=3, seed=SEED)
            frac = B.prefill_flops(model, n) / (pre["ms"] / 1e3) / (tensor * 1e12)
            print(json.dumps({"prompt_tokens": n, "ms": round(pre["ms"], 3), "tok_s": round(pre["value"], 1),
                              "tensor_frac": round(frac, 3)}), flush=True)
            del eng
            torch.cuda.empty_cache()
        return 0
    else:
        base.update(num_hidden_layers=30, full_attn_idxs=[2, 6, 10, 14, 18, 22, 25, 28], intermediate_size=10752,
                    max_position_embeddings=8192)
        cfg = Lfm2Config.from_dict(base)
        model = random_model(cfg, 4, dtype="bfloat16", device="cuda:0")
        gen = Generator(model, ctx=8192, page_size=16, n_pages=64 * 80, max_running=64, max_batch_tokens=8192, seed=4)
        pre = B.measure_prefill(gen.engine, 8000, warmup=2, runs=3, seed=4)
        dec1 = B.measure_decode(gen.engine, 1, 8000, 64, 4, seed=4)
        dec64 = B.measure_decode(gen.engine, 64, 1024, 64, 4, seed=4)
        res = {"workload": "LFM2-2.6B shape (30 layers, FFN 7168): 8,000-token prompt, greedy decode at 8k, batch 64 at 1k",
               "prefill_8000_ms": round(pre["ms"], 2), "prefill_tok_s": round(pre["value"], 1),
               "decode_b1_ctx8000_tok_s": round(dec1["tok_s"], 1), "decode_b1_gbs": round(dec1["gbs"], 1),
               "decode_b64_ctx1024_tok_s": round(dec64["tok_s"], 1), "decode_b64_gbs": round(dec64["gbs"], 1)}
    print(json.dumps({k: (round(v, 2) if isinstance(v, float) else v) for k, v in res.items()}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="float32: the engine's true 32-bit twin on the same (bfloat16-rounded) weights; "
                         "with --only prefill or --only decode (the benchmark line itself is bfloat16)")
    ap.add_argument("--skip-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--workload", choices=["serve700m", "long2p6b", "sweep", "potivik", "petelix", "sisadra", "selivik"], default=None,
                    help="run one of the other workloads instead (prints its own JSON lines); 'potivik' / 'petelix' / "
                         "'sisadra' / 'selivik': that design at layer sizes of a real model, beside an LFM2 model of equal size")
    ap.add_argument("--size", default=None, help="with --workload potivik, petelix, sisadra or selivik: '1k', '2k' or both with a comma (default both)")
    ap.add_argument("--prompt-tokens", type=int, default=None,
                    help="with --only prefill / prefill-timeline / products: another prompt length than 2,048")
    ap.add_argument("--only", default=None,
                    choices=["decode", "prefill", "timeline", "prefill-timeline", "products", "attention", "trace"],
                    help="measure one phase only (for short profiler captures; the line is then partial); "
                         "'timeline' / 'prefill-timeline': the kernels of one decode step inside its graph / of one "
                         "prompt step, from CUPTI; 'products': the prompt step's matrix products alone (with "
                         "-DGB_PAIR_TRACE: and the phases inside the CTA-pair kernel); 'attention': the prompt attention "
                         "kernel alone at 2,048 to 16,384 tokens; 'trace': time "
                         "stamps from inside a decode step's product kernels (a -DGB_GEMM_TRACE or -DGB_DECODE_TRACE build)")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm()
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)

    import torch
    from gibbs_b200 import Generator, Lfm2Config, random_model
    from gibbs_b200.engine import benchmark as B

    if a.workload in ("potivik", "petelix", "sisadra", "selivik"):
        return potivik_workload(a)
    if a.workload:
        return other_workload(a)
    raw = dict(LFM2_1P2B)
    full_layers = raw["num_hidden_layers"]
    if a.layers is not None and a.layers < full_layers:
        raw["num_hidden_layers"] = a.layers
        raw["full_attn_idxs"] = [i for i in raw["full_attn_idxs"] if i < a.layers]
    cfg = Lfm2Config.from_dict(raw)
    peaks = B.load_peaks(os.path.join(ROOT, "MEASURED_PEAKS.json"))
    torch.manual_seed(0)
    if a.dtype != "bfloat16" and a.only not in ("prefill", "decode"):
        print("bench.py: --dtype float32 goes with --only prefill or --only decode")
        return 2
    prompt_tokens = PROMPT_LEN
    if a.prompt_tokens is not None:
        if a.only not in ("prefill", "prefill-timeline", "products") or not 1 <= a.prompt_tokens <= PROMPT_LEN:
            print(f"bench.py: --prompt-tokens (1 to {PROMPT_LEN}) goes with --only prefill, prefill-timeline or products")
            return 2
        prompt_tokens = a.prompt_tokens
    if a.only == "products":
        print(B.prompt_product_times(cfg, prompt_tokens, peaks["bf16_tflops"]))
        return 0
    if a.only == "attention":
        print(B.prompt_attention_times())
        return 0
    model = random_model(cfg, SEED, dtype=a.dtype, device="cuda:0", stored_dtype=torch.bfloat16)

    page_size = 16
    max_batch = max(64, a.batch)
    gen = Generator(model, ctx=CONTEXT, page_size=page_size, n_pages=max_batch * (CONTEXT // page_size),
                    max_running=max_batch, max_batch_tokens=2048)
    eng = gen.engine

    if a.only == "prefill":
        pre = B.measure_prefill(eng, prompt_tokens, warmup=a.warmup, runs=a.steps, seed=SEED)
        print(json.dumps({"partial": "prefill", "dtype": a.dtype, "prefill": pre}))
        return 0
    if a.only == "timeline":
        print(B.format_timeline(B.decode_timeline(eng, a.batch, PROMPT_LEN, seed=SEED)))
        return 0
    if a.only == "prefill-timeline":
        print(B.format_timeline(B.prefill_timeline(eng, prompt_tokens, seed=SEED), "prompt"))
        return 0
    if a.only == "trace":
        print(B.decode_kernel_trace(eng, a.batch, PROMPT_LEN, seed=SEED))
        return 0
    if a.only == "decode":
        dec = B.measure_decode(eng, a.batch, PROMPT_LEN, a.steps, a.warmup, seed=SEED)
        print(json.dumps({"partial": "decode", "dtype": a.dtype, "decode": dec}))
        return 0
    pre = B.measure_prefill(eng, PROMPT_LEN, warmup=a.warmup, runs=5, seed=SEED)
    pre_flops = B.prefill_flops(model, PROMPT_LEN)
    pre["frac"] = pre_flops / (pre["ms"] / 1e3) / (peaks["bf16_tflops"] * 1e12)

    # as many regions as the context has room for after the prompt (five by default)
    repeats = max(1, min(REPEATS, (CONTEXT - PROMPT_LEN - a.warmup - 4 * max_batch - 32) // max(a.steps, 1)))
    with B.ClockSampler() as clocks:
        dec = B.measure_decode(eng, a.batch, PROMPT_LEN, a.steps, a.warmup, seed=SEED, repeats=repeats)
    e2e = B.measure_decode_e2e(gen, a.batch, PROMPT_LEN, a.steps, a.warmup, seed=SEED, repeats=repeats)
    points = {}
    if not a.skip_points:
        for b in (1, 64):
            if b != a.batch:
                points[f"decode_b{b}"] = round(B.measure_decode(eng, b, PROMPT_LEN, a.steps, a.warmup, seed=SEED,
                                                                 repeats=min(3, repeats))["tok_s"], 1)

    line = {
        "metric": "LFM2-1.2B decode tok/s", "value": round(dec["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(dec["ms_per_step"], 4),
        "repeats": dec["repeats"], "spread": round(dec["spread"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) seed 2, uniform-random token ids",
        "config": {
            "model": "LFM2-1.2B shape", "global_batch": a.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
            "parallelism": "none (1 GPU)", "layers": cfg.num_hidden_layers, "layers_full": full_layers,
            "attention_layers": len(cfg.attention_layers), "hidden": cfg.hidden_size,
            "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "ffn": cfg.ffn_dim, "vocab": cfg.vocab_size, "conv_L_cache": cfg.conv_L_cache, "page_size": page_size,
            "l2": "step inputs (2.3 GB of weights) exceed L2; no flush",
        },
        "e2e": {k: (round(v, 4 if k == "spread" else 1) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": dec["launches"],
        "prefill": {"value": round(pre["value"], 1), "tokens": pre["tokens"], "ms": round(pre["ms"], 3),
                    "frac": round(pre["frac"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(dec["gbs"], 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(dec["gbs"] / peaks["hbm_gbs"], 4), "peaks": peaks["source"]},
        "points": points,
        "clocks": clocks.summary(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
