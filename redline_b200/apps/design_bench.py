"""Prefill and decode throughput of one architecture beside another at equal layer sizes, with the
per-op roofline fractions of both (``bench.py --compare-design kapitar``, ``pufevik`` or ``vizotar``).

Every size is a handful of layers whose matrices have the shapes of a real model's (random weights):
the Kapitar model has one layer of every kind (attention + dense, lightning + routed, attention + routed,
lightning + dense), the Llama model beside it the same width, number of layers, heads and kv heads, a
head size equal to the width of a Kapitar head's two maps, and a gated feed-forward with as many
parameters as the dense one.  Prefill: one prompt alone through ``Engine.step_tokens`` (CUDA events around
the call, the median of the repetitions).  Decode: ``batch`` requests decoding together through
``Engine.step`` (the engine's own per-step CUDA events).  Per-op: the engine's op profiler on eager steps,
each op's bytes and operations against the measured copy bandwidth and matrix-product rate.

The Pufevik model has two layers of each kind (a pair of windowed attention with a sink beside a matrix
memory, and gated full attention with blended values; every layer with a gated feed-forward), the Llama
model beside it the same width, number of layers, heads, kv heads, head size and feed-forward width.

The Vizotar model has four layers on four residual streams: a pair (windowed attention with a sink, short
convolutions and YaRN rotation, beside a matrix memory) with a dense feed-forward, the gated delta rule with
routed experts, a pair with routed experts, the delta rule with a dense feed-forward.  Beside it stands
Pufevik, the closest architecture the package has (the same pair without convolutions on one stream, full
attention where Vizotar has the delta rule, dense feed-forwards), at the same width, heads, head sizes,
window, memory sizes and feed-forward width; the routed layers' chosen experts together are as wide as the
dense feed-forward.

The Venezen model has four layers: attention over a cached latent with a dense gated feed-forward, windowed
attention whose keys are its values with routed experts (identity experts among the router's outputs, a shared
expert), the latent attention with routed experts, the windowed attention with a dense feed-forward.  Beside
it stands Kapitar, the closest architecture the package has (layer norms, attention through the same kernels
over the same window with two score maps of half the key size, routed experts with a shared one; linear
attention where Venezen attends over latents), at the same width, heads, kv heads, window and expert count;
Venezen's gated feed-forwards have three matrices for Kapitar's two and are two thirds as wide.
"""

from __future__ import annotations

import os
import tempfile
import time
from typing import Any, Dict, List

SIZES: Dict[str, Dict[str, int]] = {
    # width, heads, kv heads, key size of one map, value size, dense width, experts, top, expert width, shared width
    "s": dict(width=1024, heads=8, kv_heads=2, dim=64, vdim=128, ff=4096, experts=16, top=4, expert_ff=512, shared_ff=1024,
              lin_dim=64, vocab=32000),
    "m": dict(width=2048, heads=16, kv_heads=4, dim=64, vdim=128, ff=8192, experts=32, top=4, expert_ff=1024, shared_ff=2048,
              lin_dim=64, vocab=32000),
}
PUFEVIK_SIZES: Dict[str, Dict[str, int]] = {
    # width, heads / kv heads / key and value size of both kinds of attention, feed-forward width, the memory's heads and sizes
    "s": dict(width=1024, heads=8, kv_heads=2, dim=128, vdim=128, ff=2816, mem_heads=8, mem_dim=64, mem_vdim=128, vocab=32000),
    "m": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, ff=5632, mem_heads=16, mem_dim=64, mem_vdim=128, vocab=32000),
}
VIZOTAR_SIZES: Dict[str, Dict[str, int]] = {
    # as PUFEVIK_SIZES, plus the delta rule's heads and sizes, the inner sizes of its low-rank projections, the experts
    "s": dict(width=1024, heads=8, kv_heads=2, dim=128, vdim=128, ff=2816, mem_heads=8, mem_dim=64, mem_vdim=128,
              delta_heads=8, delta_qk_heads=4, delta_dim=128, delta_vdim=128, rank=64, experts=16, top=4, expert_ff=704,
              streams=4, taps=4, vocab=32000),
    "m": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, ff=5632, mem_heads=16, mem_dim=64, mem_vdim=128,
              delta_heads=16, delta_qk_heads=8, delta_dim=128, delta_vdim=128, rank=128, experts=32, top=4, expert_ff=1408,
              streams=4, taps=4, vocab=32000),
}
VENEZEN_SIZES: Dict[str, Dict[str, int]] = {
    # SIZES' keys for the Kapitar model beside it, plus the latent attention's sizes (a cached row of kv_rank + rot_dim
    # entries), the gated feed-forwards' widths (two thirds of Kapitar's ungated ones) and the identity experts
    "s": dict(SIZES["s"], lat_dim=64, rot_dim=32, lat_vdim=64, kv_rank=192, gated_ff=2816, gated_expert_ff=384,
              gated_shared_ff=768, identity=2),
    "m": dict(SIZES["m"], lat_dim=64, rot_dim=32, lat_vdim=64, kv_rank=192, gated_ff=5632, gated_expert_ff=704,
              gated_shared_ff=1408, identity=4),
}
WINDOW, KEEP_FIRST = 1024, 4
PROMPT = 2048
DECODE_PROMPT = 512


def kapitar_config(s: Dict[str, int]) -> Dict[str, Any]:
    att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "diff": 0.5, "softcap": 30.0,
           "scale": s["dim"] ** -0.5, "mask": {"size": WINDOW, "keep_first": KEEP_FIRST}}
    lin = {"heads": s["heads"], "dim": s["lin_dim"], "vdim": s["vdim"],
           "decay": [1.0 - 2.0 ** -(3 + 5 * h / max(s["heads"] - 1, 1)) for h in range(s["heads"])]}
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "shared": {"ff": s["shared_ff"]},
           "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": 4, "keep": 2}}}
    return {"architecture": "Kapitar", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "layers": [{"type": "attention", "mixer": att, "mlp": dense}, {"type": "lightning", "mixer": lin, "mlp": moe},
                       {"type": "attention", "mixer": att, "mlp": moe}, {"type": "lightning", "mixer": lin, "mlp": dense}]}


def llama_config(s: Dict[str, int]) -> Dict[str, Any]:
    inter = (2 * s["ff"] // 3 + 255) // 256 * 256          # three matrices instead of two
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 4, "hidden_size": s["width"],
            "num_attention_heads": s["heads"], "num_key_value_heads": s["kv_heads"], "head_dim": 2 * s["dim"],
            "intermediate_size": inter, "vocab_size": s["vocab"], "rope_theta": 500000.0, "rope_scaling": None,
            "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192, "hidden_act": "silu"}


def pufevik_config(s: Dict[str, int]) -> Dict[str, Any]:
    heads = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "scale": s["dim"] ** -0.5}
    pair = {"left": dict(heads, mask={"size": WINDOW}, rot={"base": 1000000.0, "dims": s["dim"] // 2}), "left_scale": 0.7,
            "right": {"heads": s["mem_heads"], "dim": s["mem_dim"], "vdim": s["mem_vdim"], "gate_cap": 12.0}, "right_scale": 0.6}
    full = dict(heads, rot={"base": 10000.0, "dims": s["dim"] // 2}, v_mix=True)
    dense = {"kind": "dense", "ff": s["ff"]}
    return {"architecture": "Pufevik", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "layers": [{"type": "parallel", "mixer": pair, "mlp": dense}, {"type": "attention", "mixer": full, "mlp": dense},
                       {"type": "parallel", "mixer": pair, "mlp": dense}, {"type": "attention", "mixer": full, "mlp": dense}]}


def llama_beside_pufevik(s: Dict[str, int]) -> Dict[str, Any]:
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 4, "hidden_size": s["width"],
            "num_attention_heads": s["heads"], "num_key_value_heads": s["kv_heads"], "head_dim": s["dim"],
            "intermediate_size": s["ff"], "vocab_size": s["vocab"], "rope_theta": 500000.0, "rope_scaling": None,
            "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192, "hidden_act": "silu"}


def vizotar_config(s: Dict[str, int]) -> Dict[str, Any]:
    left = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "scale": s["dim"] ** -0.5,
            "mask": {"size": WINDOW}, "conv": s["taps"],
            "rot": {"base": 1000000.0, "dims": s["dim"] // 2,
                    "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    pair = {"left": left, "right": {"heads": s["mem_heads"], "dim": s["mem_dim"], "vdim": s["mem_vdim"], "gate_cap": 12.0}}
    delta = {"heads": s["delta_heads"], "kv_heads": s["delta_qk_heads"], "dim": s["delta_dim"], "vdim": s["delta_vdim"],
             "conv": s["taps"], "decay_rank": s["rank"], "gate_rank": s["rank"]}
    dense = {"kind": "dense", "ff": s["ff"], "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "router": {"experts": s["experts"], "top": s["top"]}}
    return {"architecture": "Vizotar", "vocab": s["vocab"], "width": s["width"], "streams": s["streams"], "norm": {"eps": 1e-6},
            "layers": [{"type": "parallel", "mixer": pair, "mlp": dense}, {"type": "channel_delta", "mixer": delta, "mlp": moe},
                       {"type": "parallel", "mixer": pair, "mlp": moe}, {"type": "channel_delta", "mixer": delta, "mlp": dense}]}


def venezen_config(s: Dict[str, int]) -> Dict[str, Any]:
    latent = {"heads": s["heads"], "dim": s["lat_dim"], "rot_dim": s["rot_dim"], "vdim": s["lat_vdim"], "kv_rank": s["kv_rank"],
              "scale": (s["lat_dim"] + s["rot_dim"]) ** -0.5, "rot": {"base": 500000.0, "dims": s["rot_dim"]}}
    key = 2 * s["dim"]                                     # Kapitar's two maps together
    windowed = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": key, "vdim": key, "scale": key ** -0.5,
                "mask": {"size": WINDOW}}
    dense = {"kind": "dense", "ff": s["gated_ff"]}
    moe = {"kind": "moe", "expert": {"ff": s["gated_expert_ff"], "limit": 7.0}, "shared": {"ff": s["gated_shared_ff"], "limit": 7.0},
           "router": {"experts": s["experts"], "identity": s["identity"], "top": s["top"], "scale": 2.5}}
    return {"architecture": "Venezen", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0},
            "layers": [{"type": "latent_attention", "mixer": latent, "mlp": dense}, {"type": "attention", "mixer": windowed, "mlp": moe},
                       {"type": "latent_attention", "mixer": latent, "mlp": moe}, {"type": "attention", "mixer": windowed, "mlp": dense}]}


# design -> (its sizes, its configuration, the architecture beside it, that one's configuration at the same sizes)
DESIGNS = {"kapitar": (SIZES, kapitar_config, "llama", llama_config),
           "pufevik": (PUFEVIK_SIZES, pufevik_config, "llama", llama_beside_pufevik),
           "vizotar": (VIZOTAR_SIZES, vizotar_config, "pufevik", pufevik_config),
           "venezen": (VENEZEN_SIZES, venezen_config, "kapitar", kapitar_config)}


def _prefill(model: str, tokens: int, reps: int, warmup: int) -> float:
    import numpy as np
    import torch
    from ..engine.engine import Engine
    eng = Engine(model, dtype="bfloat16", max_num_seqs=2, max_num_batched_tokens=tokens, max_seq_len=tokens + 16,
                 kv_cache_tokens=2 * tokens + 64, cuda_graphs=True, async_scheduling=False)
    toks = np.random.RandomState(1).randint(0, eng.vocab_size, size=tokens).tolist()
    times = []
    for i in range(warmup + reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        eng.step_tokens([("p", toks, [tokens - 1])], graphs=True)
        b.record()
        torch.cuda.synchronize()
        eng.close_request("p")
        if i >= warmup:
            times.append(a.elapsed_time(b))
    eng.runner.check_status()
    del eng
    torch.cuda.empty_cache()
    times.sort()
    return times[len(times) // 2]


def _decode(model: str, batch: int, prompt_len: int, steps: int, warmup: int) -> Dict[str, float]:
    import numpy as np
    import torch
    from ..engine.engine import Engine
    from ..sampling import SamplingParams
    new_tokens = warmup + steps + 8
    eng = Engine(model, dtype="bfloat16", max_num_seqs=batch, max_num_batched_tokens=2048,
                 max_seq_len=prompt_len + new_tokens + 16, kv_cache_tokens=batch * (prompt_len + new_tokens + 32))
    rng = np.random.RandomState(0)
    for i in range(batch):
        eng.add_request(rng.randint(0, eng.vocab_size, size=prompt_len).tolist(),
                        SamplingParams(max_new_tokens=new_tokens, ignore_eos=True, seed=i))
    eng.record_steps = True
    while not (eng.records and eng.records[-1].kind == "decode" and eng.records[-1].num_seqs == batch):
        eng.step()
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    eng.records.clear()
    launches0 = eng.runner.num_kernel_launches
    for _ in range(steps):
        eng.step()
    while len(eng.records) < steps:
        eng.step()
    torch.cuda.synchronize()
    recs = eng.records[:steps]
    gpu_ms = sum(r.gpu_ms for r in recs)
    out = {"ms_per_step": gpu_ms / steps, "tok_s": batch * steps / (gpu_ms / 1e3), "cuda_graph": all(r.cuda_graph for r in recs),
           "launches_per_step": (eng.runner.num_kernel_launches - launches0) / max(len(eng.records), 1)}
    eng.runner.check_status()
    del eng
    torch.cuda.empty_cache()
    return out


def _ops(model: str, tokens: int, batch: int, hbm_gbs: float, tflops: float) -> List[Dict[str, Any]]:
    """The per-op table of one prompt step of ``tokens`` tokens and of single-token steps of ``batch`` sequences."""
    import numpy as np
    import torch
    from ..engine.engine import Engine
    eng = Engine(model, dtype="bfloat16", max_num_seqs=batch + 1, max_num_batched_tokens=tokens, max_seq_len=tokens + 64,
                 kv_cache_tokens=(batch + 1) * (tokens + 64), cuda_graphs=False, async_scheduling=False)
    rng = np.random.RandomState(2)
    prompts = [rng.randint(0, eng.vocab_size, size=tokens).tolist() for _ in range(batch)]
    eng.step_tokens([("w", prompts[0], [tokens - 1])])             # compiles, sizes workspaces
    eng.close_request("w")
    for i in range(1, batch):                                      # contexts for the single-token steps
        eng.step_tokens([(f"d{i}", prompts[i][:DECODE_PROMPT], [])])
    eng.step_tokens([("d0", prompts[0][:DECODE_PROMPT], [])])
    eng.step_tokens([(f"d{i}", [1], [0]) for i in range(batch)])
    torch.cuda.synchronize()
    eng.set_op_profiling(True)
    for _ in range(3):
        eng.step_tokens([("w", prompts[0], [tokens - 1])])
        eng.close_request("w")
    for _ in range(8):
        eng.step_tokens([(f"d{i}", [2], [0]) for i in range(batch)])
    rows = eng.op_profile(hbm_gbs, tflops)
    eng.set_op_profiling(False)
    del eng
    torch.cuda.empty_cache()
    keep = ("op", "ms_per_pass", "calls_per_pass", "pct", "gb_s", "tflop_s", "roofline_frac")
    return [{k: (round(v, 4) if isinstance(v, float) else v) for k, v in r.items() if k in keep} for r in rows]


def compare(design: str, sizes: List[str], steps: int, warmup: int, batch: int, hbm_gbs: float, tflops: float,
            with_ops: bool = True) -> Dict[str, Any]:
    from ..config import config_from_dict
    from ..weights import write_random_model
    if design not in DESIGNS:
        raise ValueError(f"no comparison is defined for '{design}' ({', '.join(DESIGNS)})")
    table, design_config, beside, beside_config = DESIGNS[design]
    out: Dict[str, Any] = {"design": design, "beside": beside, "prompt_tokens": PROMPT, "decode_batch": batch,
                           "decode_prompt": DECODE_PROMPT, "dtype": "bf16", "data": "synthetic (random weights and tokens)",
                           "sizes": {}}
    with tempfile.TemporaryDirectory() as tmp:
        for name in sizes:
            s = table[name]
            entry: Dict[str, Any] = {"shape": dict(s, layers=4, window=WINDOW)}
            if design == "kapitar":
                entry["shape"]["keep_first"] = KEEP_FIRST
            for arch, cfg in ((design, design_config(s)), (beside, beside_config(s))):
                d = os.path.join(tmp, f"{arch}_{name}")
                t0 = time.time()
                write_random_model(d, config_from_dict(cfg), seed=0)
                ms = _prefill(d, PROMPT, reps=5, warmup=3)
                dec = _decode(d, batch, DECODE_PROMPT, steps, max(warmup, 3))
                entry[arch] = {"prefill_ms": round(ms, 3), "prefill_tok_s": round(PROMPT / (ms / 1e3)),
                               "decode_ms_per_step": round(dec["ms_per_step"], 4), "decode_tok_s": round(dec["tok_s"]),
                               "decode_cuda_graph": dec["cuda_graph"], "decode_launches_per_step": round(dec["launches_per_step"], 1),
                               "seconds": round(time.time() - t0, 1)}
                if with_ops:
                    entry[arch]["ops"] = _ops(d, PROMPT, batch, hbm_gbs, tflops)
            out["sizes"][name] = entry
    return out
