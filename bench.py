"""Benchmark of the hybrid-MoE token loop on B200: decode tok/s on the 35B-A3B-shape NVFP4 model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]

A step is one decode step (one token for each of B sequences) after a 512-token random prompt at a KV
capacity of 8192 (BASELINE.json config 3). Prints ONE JSON line: device-timed throughput (`value`), the same
through the C ABI with host buffers (`e2e`), the roofline of the dominant kernel measured live with CUDA
events, the CPU oracle timed on the host cores beside it, clocks sampled during the timed region.
With N > 1 (torchrun) the headline is expert parallelism: the routed experts sharded over the ranks, dense layers
replicated, every rank its own sequences, rows exchanged through peer memory (`expert_parallel`); the figure with a full
copy of the model per rank and no exchange at all stays beside it (`replicas`), and both again at 16 sequences per GPU.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from inferred_thoughts_b200 import configs  # noqa: E402

PROMPT, N_CTX = 512, 8192
FALLBACK_HBM = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture summarised in
# profiles/decode_step_bs1_kernels_4layer_ncu_full.md (per-launch traffic does not depend on the layer count)
NCU_TRAFFIC = {"k_moe_glu": 9503000, "k_moe_down": 5881000, "k_in_proj[gdn]": 27570000, "k_in_proj[ffn]": 4413000,
               "k_out_proj": 8943000, "k_gdn_core": 2192000}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM, "fallback 6650 GB/s (no MEASURED_PEAKS.json)"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 50 ms while the timed region runs (20 steps are about 60 ms)."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--id={device}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        import datetime
        t_stop = datetime.datetime.now()
        time.sleep(0.25)
        self.p.terminate(); self.p.wait()
        self.f.flush(); self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                # samples taken after the timed region ended (the GPU idling while this sampler is shut down) do not count
                if datetime.datetime.strptime(c[0], "%Y/%m/%d %H:%M:%S.%f") > t_stop and sm:
                    continue
            except ValueError:
                pass
            try:
                sm.append(float(c[1])); mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.f.name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def prompts(batch, seed, n_vocab):
    return np.stack([np.random.default_rng(seed + i).integers(0, n_vocab, PROMPT).astype(np.uint32) for i in range(batch)])


def bench_config(args, world):
    """The `config` object of the JSON line: what both arms (product and --impl reference) run, key for key."""
    B = args.batch
    return {"workload": f"cfg3-decode-35B-A3B-shape-bs{B}" if args.model == "m35b" else f"cfg5-decode-177B-shape-bs{B}",
            "batch_per_gpu": B, "prompt": PROMPT, "n_ctx": N_CTX, "kv": "bf16", "parallelism": "replicas" if world > 1 else "single",
            "l2": "each step streams ~2.8 GB of weights, far beyond the 126 MB L2; no flush needed",
            **({"layers": args.layers, "not_a_bench_number": True} if args.layers else {})}


def load_oracle(model, dims, seed):
    """The CPU oracle (C++ restatement of the reference CPU path) holding the same weights, copied back from the device
    generator (bit-identical to the CPU generator, and minutes faster for 35 B parameters)."""
    from oracle import oracle_py as O
    om = O.OracleModel(O.ModelDims(**dims))
    t0 = time.time()
    for s in om.specs:
        data, sc = model.synth_read(seed, s["name"], s["bytes"], s["n_expert"] if s["has_scale"] else 0)
        om.set_tensor(s["name"], data, sc)
    return om, time.time() - t0


def cpu_decode_tok_s(om, dims, seed, threads, prompt, warmup, steps, budget_s=None):
    """Decode tokens on the CPU oracle after the same `prompt` the product arm uses, KV in bf16 as there. Timed: `steps`
    greedy tokens (cut short after `budget_s` seconds when given); untimed: the prompt pass and `warmup` tokens."""
    from oracle import oracle_py as O
    O.lib().orc_set_threads(threads)
    om.begin(len(prompt) + warmup + steps + 8, kv_bf16=True)
    t0 = time.perf_counter()
    tok = int(np.argmax(om.forward(prompt)))
    prefill_s = time.perf_counter() - t0
    for _ in range(warmup):
        tok = int(np.argmax(om.forward([tok])))
    n, t0 = 0, time.perf_counter()
    while n < steps:
        tok = int(np.argmax(om.forward([tok]))); n += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return n / dt, n, dt, prefill_s


def parity_check(host, model, om, dims, seed, mode, n_prompt=16, n_new=16):
    """The timed path against the CPU oracle IN THE BENCH'S OWN MODE (`mode`: the ops string of the timed engine): a short
    prompt in one multi-row pass, then n_new teacher-forced decode steps through the fused one-token step (the oracle's
    greedy token goes to both sides, tests/cuda_ops.rs:544-626 in the reference). Reports whether every greedy choice agrees,
    the first divergence with the oracle's top-2 margin there (src/profile.rs:88-93), routing-id mismatches over every
    layer and step, and the logit distance."""
    from oracle import oracle_py as O
    O.lib().orc_set_threads(O.lib().orc_hw_threads())
    L, K = dims["n_layer"], dims["n_expert_used"]
    prompt = np.random.default_rng(seed + 11).integers(0, dims["n_vocab"], n_prompt).astype(np.uint32)
    eng = host.Engine(model, n_prompt + n_new + 8, 1)
    om.begin(n_prompt + n_new + 8, kv_bf16="kv=bf16" in mode, log_routes=True)
    o = om.forward(prompt); g = eng.prefill(prompt)
    mism = int((eng.read_routes(L, K)[:, 0, :] != om.route_log().reshape(L, n_prompt, K)[:, -1, :]).sum())
    compared = L * K
    first_div, margin, max_abs, min_cos = None, None, 0.0, 1.0
    for step in range(n_new + 1):
        max_abs = max(max_abs, float(np.abs(o - g).max()))
        a, b = o.astype(np.float64), g.astype(np.float64)
        min_cos = min(min_cos, float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300)))
        t = int(np.argmax(o))
        if int(np.argmax(g)) != t and first_div is None:
            top2 = np.partition(o, -2)[-2:]
            first_div, margin = step, float(top2[1] - top2[0])
        if step == n_new:
            break
        om.clear_route_log()
        o = om.forward([t])
        lg, _ = eng.decode([t]); g = lg[0]
        mism += int((eng.read_routes(L, K)[:, 0, :] != om.route_log().reshape(L, K)).sum()); compared += L * K
    eng.close()
    return {"mode": mode, "against": "CPU oracle (port of the reference CPU path), same weights", "prompt": n_prompt, "tokens": n_new + 1,
            "tokens_equal": first_div is None, "first_divergence": first_div, "oracle_top2_margin_at_divergence": margin,
            "routing_id_mismatches": mism, "routing_ids_compared": compared, "logits_max_abs": max_abs, "logits_min_cosine": min_cos}


def kernel_breakdown(eng, tok):
    from inferred_thoughts_b200 import host  # noqa: F401

    class Stat(C.Structure):
        _fields_ = [("name", C.c_char * 32), ("launches", C.c_uint32), ("ms", C.c_float), ("bytes", C.c_uint64)]
    arr = (Stat * 16)()
    n = C.c_size_t()
    t = np.ascontiguousarray(tok, np.uint32)
    acc = {}
    reps = 3
    for _ in range(reps):
        if eng.L.itb_engine_profile_step(eng.h, C.c_void_p(t.ctypes.data), arr, C.c_size_t(16), C.byref(n)):
            eng.model.ops.check(); raise RuntimeError("profile_step failed")
        for i in range(n.value):
            a = acc.setdefault(arr[i].name.decode(), [0, 0.0, 0])
            a[0] += arr[i].launches; a[1] += arr[i].ms; a[2] += arr[i].bytes
    out = []
    for name, (launches, ms, nbytes) in acc.items():
        if launches:
            out.append(dict(kernel=name, launches_per_step=launches // reps, ms_per_step=ms / reps, bytes_per_step=nbytes // reps,
                            gbs=nbytes / ms / 1e6 if ms > 0 else None))
    return sorted(out, key=lambda k: -k["ms_per_step"])


def experts_microbench(host, ops, hbm):
    """BASELINE config 2: the routed-expert matmuls alone (gate+up with SiLU, then down) at hidden 2048, expert FFN 512,
    256 experts, top-8, Zipf(1.1)-skewed routing, through the op-level seam with buffers resident on the device
    (`moe_glu` + `matmul_experts`, src/ops/mod.rs:1049-1117). Weights are random valid NVFP4 blocks."""
    import torch
    H, ff, E, K = 2048, 512, 256, 8
    rng = np.random.default_rng(2)

    def blocks(n_out, n_in):
        nb = E * n_out * n_in // 64
        b = np.zeros((nb, 36), np.uint8)
        b[:, :4] = rng.integers(0x20, 0x50, (nb, 4)); b[:, 4:] = rng.integers(0, 256, (nb, 32))
        return b.reshape(-1), ((rng.random(E).astype(np.float32) + 0.5) * 0.3)
    (gb, gs), (ub, us), (db, ds) = blocks(ff, H), blocks(ff, H), blocks(H, ff)
    G, U, D = host.Experts(gb, host.NVFP4, H, ff, E, gs), host.Experts(ub, host.NVFP4, H, ff, E, us), host.Experts(db, host.NVFP4, ff, H, E, ds)
    base = (-1.1 * np.log(np.arange(1, E + 1))).astype(np.float32)
    out = {}
    for T in (1, 8, 32, 512, 8192):
        x = rng.standard_normal(T * H).astype(np.float32)
        lg = np.concatenate([base[rng.permutation(E)] for _ in range(T)]).astype(np.float32)
        e = np.exp(lg.reshape(T, E) - lg.reshape(T, E).max(1, keepdims=True)); probs = (e / e.sum(1, keepdims=True)).astype(np.float32).reshape(-1)
        h = np.zeros(T * K * ff, np.float32); scratch = np.zeros_like(h); o = np.zeros(T * K * H, np.float32)
        ops.begin_pass(T)
        route = ops.route(probs, E, K)
        ids, _ = ops.read_route(route)
        for _ in range(2):
            ops.moe_glu(G, U, route, x, h, scratch); ops.matmul_experts(D, route, h, o)
        ops.check(); torch.cuda.synchronize()
        iters = 50 if T <= 32 else 10 if T <= 512 else 3
        t0 = time.perf_counter()
        for _ in range(iters):
            ops.moe_glu(G, U, route, x, h, scratch); ops.matmul_experts(D, route, h, o)
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) / iters * 1e3
        ops.check()
        distinct = len(set(ids.tolist()))
        by = distinct * 3 * (H * ff // 64 * 36) + T * H * 4 + T * K * (ff + H) * 4
        out[str(T)] = {"ms": ms, "tok_per_s": T / (ms / 1e3), "distinct_experts": distinct, "algorithmic_GBs": by / ms / 1e6,
                       "frac_of_hbm": by / ms / 1e6 / hbm, "int8_TOPS": 2.0 * T * K * 3 * H * ff / (ms / 1e3) / 1e12}
    # the same matmuls as FP4 x FP4 block-scaled tensor-core GEMMs (tcgen05.mma kind::mxf4nvf4), against the measured ceiling of
    # that instruction on this GPU
    tc = host.B200Ops(0, "experts=fp4tc")
    try:
        peak = max(tc.fp4_ceiling(n=128)[0], tc.fp4_ceiling(n=256)[0])
        fp4 = {"fp4_peak_TFLOPs_measured": peak, "peak_method": "back-to-back tcgen05.mma kind::mxf4nvf4 on unchanging shared-memory operands, one block per SM, accumulators verified"}
        for T in (512, 2048, 8192, 32768):
            x = rng.standard_normal(T * H).astype(np.float32)
            lg = np.concatenate([base[rng.permutation(E)] for _ in range(T)]).astype(np.float32)
            e = np.exp(lg.reshape(T, E) - lg.reshape(T, E).max(1, keepdims=True)); probs = (e / e.sum(1, keepdims=True)).astype(np.float32).reshape(-1)
            h = np.zeros(T * K * ff, np.float32); scratch = np.zeros_like(h); o = np.zeros(T * K * H, np.float32)
            tc.begin_pass(T)
            route = tc.route(probs, E, K)
            for _ in range(2):
                tc.moe_glu(G, U, route, x, h, scratch); tc.matmul_experts(D, route, h, o)
            tc.check(); torch.cuda.synchronize()
            iters = 10 if T <= 2048 else 3
            t0 = time.perf_counter()
            for _ in range(iters):
                tc.moe_glu(G, U, route, x, h, scratch); tc.matmul_experts(D, route, h, o)
            torch.cuda.synchronize()
            ms = (time.perf_counter() - t0) / iters * 1e3
            tc.check()
            tf = 2.0 * T * K * 3 * H * ff / (ms / 1e3) / 1e12
            fp4[str(T)] = {"ms": ms, "tok_per_s": T / (ms / 1e3), "fp4_TFLOPs": tf, "frac_of_fp4_peak": tf / peak}
        out["fp4_tensor_cores"] = fp4
    finally:
        tc.close()
    return out


def tiered_decode(host, ops, dims, seed, frac=0.5, steps=32):
    """Batch-1 decode with the routed experts in pinned host memory and `frac` of the (layer, expert) entries cached in HBM
    under GCLOCK (uniform-random routing of the synthetic router: a worst case for any cache)."""
    cold = host.Model(ops, host.ModelDims(**dims)); cold.synth(seed); cold.offload_experts()
    cap = int(dims["n_layer"] * dims["n_expert"] * frac)
    eng = host.Engine(cold, N_CTX, 1, tier_capacity=cap)
    eng.prefill(prompts(1, seed + 5, dims["n_vocab"]), want_logits=False)
    first = eng.decode_loop(np.zeros(1, np.uint32), 4)[-1]
    s0 = eng.tier_stats()
    eng.decode_loop(first, steps)
    ms = eng.last_ms() / steps
    s1 = eng.tier_stats()
    hits, misses = s1["hits"] - s0["hits"], s1["misses"] - s0["misses"]
    out = {"value": 1e3 / ms, "unit": "tok/s", "ms_per_step": ms, "pool_entries": cap, "pool_fraction": frac,
           "hit_rate": hits / max(1, hits + misses), "host_to_hbm_MB_per_token": (s1["bytes_moved"] - s0["bytes_moved"]) / steps / 1e6}
    eng.close(); cold.close()
    return out


FAST_MODE = "kv=bf16,exact=0,experts=fp4tc,dense=f16tc"
FAST_MODE_Q8 = "kv=bf16,exact=0,experts=fp4tc,dense=q8tc"
PREFILL_ROWS = 2048


def timed_prefill(host, model, n_vocab, seed, n=5548):
    """One n-token prompt through passes of PREFILL_ROWS rows (device time by CUDA events inside the library)."""
    os.environ["ITB_ROWS"] = str(PREFILL_ROWS)
    try:
        eng = host.Engine(model, N_CTX, 1)
    finally:
        del os.environ["ITB_ROWS"]
    pr = np.random.default_rng(seed + 7).integers(0, n_vocab, n).astype(np.uint32)
    eng.prefill(pr[:256], want_logits=False); eng.reset()          # warm-up: first-use work (operand images of the weights, scratch)
    eng.prefill(pr, want_logits=False)
    ms = eng.last_ms()
    eng.close()
    return ms


def other_configs(host, model, dims, seed, hbm, args, mode):
    """The other halves of the metric on the same shape: the 5,548-token prefill (BASELINE config 4) and batch-32 decode
    (config 3), each with its own roofline fraction; and the tolerance-class arithmetic (FP4 x FP4 tensor-core experts, tensor-core
    attention, chunk-parallel delta rule, tree-summed F32 dots) on a second copy of the model, for the prefill and for batch-1
    decode, beside the bit-exact numbers."""
    out = {}
    n_vocab = dims["n_vocab"]
    flop_tok = 2.0 * dims["n_layer"] * dims["n_expert_used"] * 3 * dims["n_embd"] * dims["expert_ff"]
    try:
        ms = timed_prefill(host, model, n_vocab, seed)
        out["prefill_5548_exact"] = {"value": 5548 / (ms / 1e3), "unit": "tok/s", "ms": ms, "rows_per_pass": PREFILL_ROWS, "ops": mode,
                                     "note": "bit-identical to the CPU path: dense Q8_0 matmuls as tcgen05 int8 MMAs with the block scales applied in CPU order, "
                                             "expert-grouped NVFP4 x int8 tiles, CPU-order attention and delta-rule scan"}
    except Exception as ex:
        out["prefill_5548_exact"] = {"error": str(ex)}
    try:
        B = 32
        eng = host.Engine(model, N_CTX, B)
        pr = np.stack([np.random.default_rng(seed + i).integers(0, n_vocab, PROMPT).astype(np.uint32) for i in range(B)])
        eng.prefill(pr, want_logits=False)
        first = eng.decode_loop(np.zeros(B, np.uint32), 4)[-1]
        steps = 32
        eng.decode_loop(first, steps)
        ms = eng.last_ms() / steps
        # distinct experts per layer from this run's routing (the last step's ids, every layer), not a formula
        K = dims["n_expert_used"]
        routes = eng.read_routes(dims["n_layer"], K)
        per_layer = [len(set(routes[il].reshape(-1).tolist())) for il in range(dims["n_layer"])]
        distinct = int(round(float(np.mean(per_layer))))
        by = model.decode_bytes(B, eng.pos(0), distinct)
        out["decode_bs32"] = {"value": B / (ms / 1e3), "unit": "tok/s", "ms_per_step": ms, "algorithmic_bytes_per_step": by, "ops": mode,
                              "frac_of_hbm": by / ms / 1e6 / hbm, "distinct_experts_per_layer_measured": {"mean": float(np.mean(per_layer)), "min": min(per_layer), "max": max(per_layer)}}
        eng.close()
    except Exception as ex:
        out["decode_bs32"] = {"error": str(ex)}
    fast_ops = fast_model = None
    try:
        fast_ops = host.B200Ops(0, FAST_MODE)
        fast_model = host.Model(fast_ops, host.ModelDims(**dims)); fast_model.synth(configs.SEEDS[args.model])
        ms = timed_prefill(host, fast_model, n_vocab, seed)
        peak = max(fast_ops.fp4_ceiling(n=128)[0], fast_ops.fp4_ceiling(n=256)[0])
        out["prefill_5548"] = {"value": 5548 / (ms / 1e3), "unit": "tok/s", "ms": ms, "rows_per_pass": PREFILL_ROWS, "ops": FAST_MODE,
                               "expert_flop_per_token": flop_tok, "expert_TFLOPs_if_the_whole_pass_were_experts": flop_tok * 5548 / (ms / 1e3) / 1e12,
                               "fp4_peak_TFLOPs_measured": peak,
                               "note": "tolerance class: routed experts as FP4 x FP4 tcgen05 block-scaled GEMMs, causal attention as 16-bit matrix products, "
                                       "chunk-parallel delta rule; dense Q8_0 matmuls as f16 tcgen05 GEMMs over dequantised operands (2^-12 per operand), small F32 "
                                       "matrices as fused-multiply-add tiles. On this random-weight model the dense rounding is past the router's margins: picks flip, "
                                       "so logits are held to a sanity bound only (tests); prefill_5548_exact_dense keeps the dense results bit-exact"}
        eng = host.Engine(fast_model, N_CTX, 1)
        eng.prefill(prompts(1, seed, n_vocab), want_logits=False)
        first = eng.decode_loop(np.zeros(1, np.uint32), 8)[-1]
        eng.decode_loop(first, 64)
        ms1 = eng.last_ms() / 64
        by = fast_model.decode_bytes(1, eng.pos(0), dims["n_expert_used"])
        out["decode_bs1_tree_dots"] = {"value": 1e3 / ms1, "unit": "tok/s", "ms_per_step": ms1, "ops": FAST_MODE, "frac_of_hbm": by / ms1 / 1e6 / hbm,
                                       "note": "the one-token step with F32 dots as lane-strided partial sums and a shuffle tree instead of the CPU's serial order: rounding-level "
                                               "differences, which on this synthetic model change greedy tokens within a few steps (see tests); the headline runs exact=1"}
        eng.close()
    except Exception as ex:
        out.setdefault("prefill_5548", {"error": str(ex)})
    finally:
        if fast_model is not None:
            fast_model.close()
        if fast_ops is not None:
            fast_ops.close()
    # the same tolerance-class pass with the dense matmuls kept bit-exact (int8 MMAs, scales in CPU order)
    fast_ops = fast_model = None
    try:
        fast_ops = host.B200Ops(0, FAST_MODE_Q8)
        fast_model = host.Model(fast_ops, host.ModelDims(**dims)); fast_model.synth(configs.SEEDS[args.model])
        ms = timed_prefill(host, fast_model, n_vocab, seed)
        out["prefill_5548_exact_dense"] = {"value": 5548 / (ms / 1e3), "unit": "tok/s", "ms": ms, "rows_per_pass": PREFILL_ROWS, "ops": FAST_MODE_Q8,
                                           "note": "as prefill_5548, but the dense Q8_0 matmuls as tcgen05 int8 MMAs per 32-element block with the scales applied in CPU "
                                                   "order (bit-identical dense results)"}
    except Exception as ex:
        out["prefill_5548_exact_dense"] = {"error": str(ex)}
    finally:
        if fast_model is not None:
            fast_model.close()
        if fast_ops is not None:
            fast_ops.close()
    return out


def expert_parallel(host, ops, model, dims, seed, args, rank, world, dist, torch):
    """The same decode workload with the routed experts sharded over the ranks (each rank: its expert range, the dense
    layers replicated, its own sequences; per MoE layer an all-gather and a reduce-scatter over NCCL). Every rank runs
    this in lockstep; returns the whole-job figure (max time over ranks)."""
    B = args.batch
    uid = host.share_unique_id(rank)
    lo, hi = host.expert_range(rank, world, dims["n_expert"])
    shard = host.Model(ops, host.ModelDims(**dims)); shard.synth(seed, lo, hi)
    eng = host.Engine(shard, N_CTX, B, ep=(rank, world, uid))
    eng.prefill(prompts(B, seed + 1000 * rank, dims["n_vocab"]), want_logits=False)
    first = eng.decode_loop(np.zeros(B, np.uint32), max(args.warmup, 3))[-1]
    dist.barrier(); torch.cuda.synchronize()
    eng.decode_loop(first, args.steps)
    torch.cuda.synchronize()
    dev_ms = eng.last_ms()
    # end to end through the C ABI: host token ids in, host argmax ids out, every step
    cur = np.zeros(B, np.uint32)
    dist.barrier(); torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        _, cur = eng.decode(cur, want_logits=False)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    # a many-row pass per rank: the packed all-to-all dispatch/combine (each rank its own 2,048-token prompt)
    pre_ms = None
    if not args.no_extra:
        os.environ["ITB_ROWS"] = str(PREFILL_ROWS)
        try:
            pe = host.Engine(shard, N_CTX, 1, ep=(rank, world, host.share_unique_id(rank)))
        finally:
            del os.environ["ITB_ROWS"]
        pr = np.random.default_rng(seed + 77 + rank).integers(0, dims["n_vocab"], PREFILL_ROWS).astype(np.uint32)
        pe.prefill(pr[:256], want_logits=False); pe.reset()
        dist.barrier(); torch.cuda.synchronize()
        pe.prefill(pr, want_logits=False)
        pre_ms = pe.last_ms()
        pe.close()
    # the same comparison at 16 sequences per GPU, where the expert kernels' weight traffic (a rank streams only its shard's
    # experts, for every rank's rows) starts to pay for the exchange: expert parallel against a full copy per GPU
    ms16, tr16 = [0.0, 0.0], []
    if not args.no_extra:
        B16, S16 = 16, 16

        def steps16(m, ep):
            e = host.Engine(m, N_CTX, B16, ep=ep) if ep else host.Engine(m, N_CTX, B16)
            try:
                pr = np.stack([np.random.default_rng(seed + 1000 * rank + i).integers(0, dims["n_vocab"], PROMPT).astype(np.uint32) for i in range(B16)])
                e.prefill(pr, want_logits=False)
                f = e.decode_loop(np.zeros(B16, np.uint32), S16)[-1]
                dist.barrier(); torch.cuda.synchronize()
                e.decode_loop(f, S16)
                if ep:
                    tr16.append(e.ep_step_transport())
                return e.last_ms() / S16
            finally:
                e.close()
        try:      # a failure here is a set-up failure common to all ranks (the ranks agree before anything is enqueued): keep the figures above
            ms16 = [steps16(shard, (rank, world, host.share_unique_id(rank))), steps16(model, None)]
        except Exception:
            ms16 = [0.0, 0.0]
    t = torch.tensor([dev_ms, e2e_s, pre_ms or 0.0, ms16[0], ms16[1]], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_s, pre_ms, ms16 = float(t[0]), float(t[1]), float(t[2]), [float(t[3]), float(t[4])]
    n_moe = dims["n_layer"]
    transport = eng.ep_step_transport()
    out = {"value": world * B * args.steps / (ms / 1e3), "unit": "tok/s", "ms_per_step": ms / args.steps, "batch_per_gpu": B,
           "e2e_tok_s": world * B * args.steps / e2e_s,
           "experts_per_gpu": hi - lo, "launches_per_step": int(eng.launches_per_step()), "step_transport": transport,
           "collectives_per_step": 0 if transport == "peer-memory" else 2 * n_moe,
           "note": "experts sharded by range, dense replicated, every rank its own sequences; one-token steps per MoE layer: " +
                   ("each rank's row and router logits stored into every rank's memory over NVLink and the served picks' rows stored straight into their "
                    "owner's memory by the expert kernels (own kernels, flags with bounded waits, no collective call)" if transport == "peer-memory" else
                    "all-gather(rows, routing) + exact-sum reduce-scatter(pair outputs) over NCCL") +
                   ", captured in the step's CUDA graph; many-row passes: packed all-to-all dispatch and combine"}
    if pre_ms:
        out["prefill_2048_per_rank"] = {"value": world * PREFILL_ROWS / (pre_ms / 1e3), "unit": "tok/s", "ms": pre_ms, "dispatch": "packed all-to-all (NCCL send/recv sized by exchanged counts)"}
    if ms16[0] > 0 and ms16[1] > 0:
        out["batch16_per_gpu"] = {"expert_parallel": {"value": world * 16 / (ms16[0] / 1e3), "unit": "tok/s", "ms_per_step": ms16[0]},
                                  "replicas": {"value": world * 16 / (ms16[1] / 1e3), "unit": "tok/s", "ms_per_step": ms16[1]},
                                  "step_transport": tr16[0] if tr16 else None,
                                  "note": "decode steps of 16 sequences per GPU (512-token prompts), device time, max over ranks; peer-memory: every rank's rows and "
                                          "routing ids stored into every rank's memory, each served pair's output row stored into its owner's memory, flags with "
                                          "bounded waits (own kernels inside the step's CUDA graph); nccl: all-gather + zero-filled exact-sum reduce-scatter"}
    eng.close(); shard.close()
    return out


def run_product(args, rank, world):
    from inferred_thoughts_b200 import host
    import torch
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank))))
    device = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(device)
    dims = dict(configs.L177B if args.model == "l177b" else configs.M35B)
    if args.layers:
        dims = configs.with_layers(dims, args.layers)   # profiling aid only: a line with "layers" set is not a bench number
    seed = configs.SEEDS[args.model]
    kv = "bf16"
    mode = f"kv={kv},exact={args.exact}" + (",dense=q8tc" if args.exact else "")
    ops = host.B200Ops(device, mode)
    model = host.Model(ops, host.ModelDims(**dims))
    t0 = time.time()
    model.synth(seed)
    synth_s = time.time() - t0
    B = args.batch
    eng = host.Engine(model, N_CTX, B)
    pr = prompts(B, seed + 1000 * rank, dims["n_vocab"])
    eng.prefill(pr, want_logits=False)
    first = np.zeros(B, np.uint32)
    # warm-up (also builds the graph): W steps
    if args.warmup:
        first = eng.decode_loop(first, args.warmup)[-1]
    # ---- device-timed region: K steps, inputs resident in HBM ----
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(device) if rank == 0 else None
    torch.cuda.profiler.start()     # a profiler run with --profile-from-start off sees exactly the timed steps
    toks = eng.decode_loop(first, args.steps)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    dev_ms = eng.last_ms()
    # ---- end to end through the C ABI: host token in, host token out, every step ----
    cur = toks[-1].copy()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        _, cur = eng.decode(cur, want_logits=False)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if sampler else None
    if dist is not None:
        t = torch.tensor([dev_ms, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_s = float(t[0]), float(t[1])
    n_pos = eng.pos(0)
    ep = None
    if world > 1 and not args.no_extra and dims["n_expert"] % world == 0:
        try:
            ep = expert_parallel(host, ops, model, dims, seed, args, rank, world, dist, torch)
        except Exception as ex:   # every rank takes the same branch: failures here are set-up failures common to all
            ep = {"error": str(ex)}
    if rank != 0:
        return
    hbm, hbm_src = peaks()
    kb = kernel_breakdown(eng, cur) if B == 1 else kernel_breakdown(host.Engine(model, 256, 1), [1])
    dom = kb[0]
    per_launch_bytes = dom["bytes_per_step"] / dom["launches_per_step"]
    per_launch_ms = dom["ms_per_step"] / dom["launches_per_step"]
    achieved = per_launch_bytes / per_launch_ms / 1e6
    step_bytes = model.decode_bytes(B, n_pos, min(dims["n_expert"], dims["n_expert_used"] * B))
    ms_per_step = dev_ms / args.steps
    value = world * B * args.steps / (dev_ms / 1e3)
    line = {
        "metric": "decode tok/s, 35B-A3B-shape NVFP4 (BASELINE.json config 3)" if args.model == "m35b" else "decode tok/s, ~177B-shape NVFP4 (BASELINE.json config 5)", "value": value, "unit": "tok/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8 (int8 x int8 / e2m1 x int8 dots, f32 accumulate; f32 state)",
        "data": "synthetic (seeded Gaussian weights quantised to NVFP4 / Q8_0, uniform-random token ids)",
        "config": bench_config(args, world),
        "run": {"n_pos_at_end": n_pos, "f32_dots": "serial-k" if args.exact else "tree", "ops": mode},
        "e2e": {"value": world * B * args.steps / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B,
                "api": "itb_engine_decode (host token ids in, host argmax ids out)"},
        "gpu_launches": int(eng.launches_per_step()) * args.steps * 2,
        "roofline": {"bound": "hbm", "kernel": dom["kernel"], "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                     "traffic": NCU_TRAFFIC.get(dom["kernel"]), "peak_source": hbm_src, "bytes_per_launch": per_launch_bytes, "ms_per_launch": per_launch_ms},
        "step_roofline": {"algorithmic_bytes_per_step": step_bytes, "achieved": step_bytes / ms_per_step / 1e6, "peak": hbm, "unit": "GB/s",
                          "frac": step_bytes / ms_per_step / 1e6 / hbm, "frac_of_8TBs_nominal": step_bytes / ms_per_step / 1e6 / 8000.0},
        "kernels": kb, "clocks": clocks, "synth_s": synth_s,
    }
    if ep is not None and "error" not in ep:
        # more than one GPU: expert parallelism is the headline (the north star reports 2/4/8 GPUs in that mode); the
        # full-copy-per-GPU figure measured above stays beside it
        line["replicas"] = {"value": line["value"], "unit": "tok/s", "ms_per_step": line["ms_per_step"], "e2e_tok_s": line["e2e"]["value"],
                            "note": "every rank a full copy of the model and its own sequences, no collective on the data path"}
        line["value"] = ep["value"]; line["ms_per_step"] = ep["ms_per_step"]
        line["e2e"]["value"] = ep["e2e_tok_s"]
        line["config"]["parallelism"] = f"ep{world} (routed experts sharded by range, dense replicated)"
        line["step_roofline"] = {"note": "per-GPU bytes differ by rank under expert parallelism (each rank streams the experts ITS pairs and its peers' pairs pick from its shard); "
                                         "see replicas for the single-GPU roofline of the same step"}
        line["expert_parallel"] = ep
    elif ep is not None:
        line["expert_parallel"] = ep
    if world == 1 and not args.no_extra:
        line["other_configs"] = other_configs(host, model, dims, seed, hbm, args, mode)
        try:
            line["other_configs"]["tiered_experts_half_in_hbm"] = tiered_decode(host, ops, dims, seed)
        except Exception as ex:
            line["other_configs"]["tiered_experts_half_in_hbm"] = {"error": str(ex)}
        try:
            line["other_configs"]["experts_microbench_cfg2"] = experts_microbench(host, ops, hbm)
        except Exception as ex:
            line["other_configs"]["experts_microbench_cfg2"] = {"error": str(ex)}
    if world == 1 and not args.no_cpu:
        om = None
        try:
            from oracle import oracle_py as O
            threads = O.lib().orc_hw_threads()
            om, load_s = load_oracle(model, dims, seed)
            line["parity"] = parity_check(host, model, om, dims, seed, mode)
        except Exception as ex:
            line["parity"] = {"error": str(ex)}
        try:
            if om is None:
                raise RuntimeError("the oracle could not be loaded")
            # bounded sample: the first 32 tokens of the prompt only (the CPU needs ~0.4 s per prompt token; `--impl reference`
            # runs the whole 512-token prompt), then decode tokens for about --cpu-budget seconds
            v, n, dt, prefill_s = cpu_decode_tok_s(om, dims, seed, threads, pr[0][:32], 1, 48, args.cpu_budget)
            line["cpu_baseline"] = {"value": v, "unit": "tok/s", "cores": threads, "kind": "port",
                                    "sample": f"{n} decode tokens ({dt:.1f} s) after the first 32 tokens of the same prompt (CPU prompt pass {prefill_s:.0f} s, untimed), "
                                              f"same weights (copied back from the device in {load_s:.0f} s), batch 1, bf16 KV"}
        except Exception as ex:  # the baseline is a report, never a reason to lose the measurement
            line["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": 0, "kind": "port", "sample": f"failed: {ex}"}
    emit(line)
    eng.close(); model.close(); ops.close()


def run_reference(args, rank, world):
    """The reference's CPU path (its algorithm, restated in C++: the reference itself is Rust and cannot be built here)
    on the host cores, on the product arm's config and metric: the same 512-token prompt (seed and all), bf16 KV, then
    `warmup` untimed and `steps` timed greedy decode tokens. The weights come from the library's device generator when a GPU
    is there -- outside the timed region, and tested equal to the CPU generator byte for byte -- else from the CPU generator."""
    if rank != 0:
        return
    from oracle import oracle_py as O
    dims = dict(configs.L177B if args.model == "l177b" else configs.M35B)
    if args.layers:
        dims = configs.with_layers(dims, args.layers)
    seed = configs.SEEDS[args.model]
    threads = O.lib().orc_hw_threads()
    src = "cpu generator"
    om = None
    try:
        from inferred_thoughts_b200 import host
        ops = host.B200Ops(0)
        model = host.Model(ops, host.ModelDims(**dims))
        om, _ = load_oracle(model, dims, seed)
        model.close(); ops.close()
        src = "device generator, copied to the host"
    except Exception:
        om = O.OracleModel(O.ModelDims(**dims))
        om.synth(seed, threads)
    pr = prompts(args.batch, seed, dims["n_vocab"])[0]        # rank 0's first sequence, as in the product arm
    v, n, dt, prefill_s = cpu_decode_tok_s(om, dims, seed, threads, pr, args.warmup, args.steps)
    emit({
        "impl": "reference", "metric": "decode tok/s, 35B-A3B-shape NVFP4 (BASELINE.json config 3)" if args.model == "m35b" else "decode tok/s, ~177B-shape NVFP4 (BASELINE.json config 5)",
        "value": v, "unit": "tok/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / n * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8 (int8 x int8 / e2m1 x int8 dots, f32 accumulate; f32 state)",
        "data": f"synthetic (seeded Gaussian weights quantised to NVFP4 / Q8_0, uniform-random token ids; weights from the {src})",
        "config": bench_config(args, world),
        "run": {"n_pos_at_end": len(pr) + args.warmup + n, "f32_dots": "serial-k", "prompt_pass_s": prefill_s},
        "cpu_baseline": {"value": v, "unit": "tok/s", "cores": threads, "kind": "port",
                         "sample": f"{n} decode tokens after the {len(pr)}-token prompt and {args.warmup} warm-up tokens, one sequence"},
        "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })


def run_probe(args):
    """One pass of the engine inside a CUDA profiler range (for `ncu --profile-from-start off`), on the benchmark's shape with
    --layers layers (default 8: about 5 GB on the device, small enough for a multi-pass capture). Prints the pass's device
    time to stderr; never a bench line."""
    import torch
    from inferred_thoughts_b200 import host
    mode, _, n = args.probe.partition(":")
    n = int(n or 1)
    dims = configs.with_layers(dict(configs.L177B if args.model == "l177b" else configs.M35B), args.layers or 8)
    ops = host.B200Ops(0, f"kv=bf16,exact={args.exact}" + ("," + args.opts if args.opts else ""))
    rng = np.random.default_rng(3)
    model = None
    if mode != "experts":
        model = host.Model(ops, host.ModelDims(**dims)); model.synth(configs.SEEDS[args.model])
    if mode == "decode":
        eng = host.Engine(model, args.probe_ctx, n)
        eng.prefill(rng.integers(0, dims["n_vocab"], (n, args.probe_prompt)).astype(np.uint32), want_logits=False)
        t = eng.decode_loop(np.zeros(n, np.uint32), max(2, args.probe_steps))[-1]
        torch.cuda.synchronize(); torch.cuda.profiler.start()
        eng.decode_loop(t, args.probe_steps)
        torch.cuda.synchronize(); torch.cuda.profiler.stop()
        if args.probe_steps > 1:
            print(f"per step: {eng.last_ms() / args.probe_steps:.3f} ms", file=sys.stderr)
    elif mode == "prefill":
        eng = host.Engine(model, max(2048, n + 64), 1)
        pr = rng.integers(0, dims["n_vocab"], n).astype(np.uint32)
        eng.prefill(pr[:min(n, 256)], want_logits=False); eng.reset()       # warm-up: first-use work (operand images of the weights, scratch) happens here
        torch.cuda.synchronize(); torch.cuda.profiler.start()
        eng.prefill(pr, want_logits=False)
        torch.cuda.synchronize(); torch.cuda.profiler.stop()
    elif mode in ("step", "timeline"):
        eng = host.Engine(model, max(2048, n + 64), 1)
        eng.prefill((np.arange(n, dtype=np.uint32) * 7919) % dims["n_vocab"], want_logits=False)
        t = eng.decode_loop([1], 8)[-1]
        if mode == "timeline":
            print_timeline(eng, dims, t)
        else:
            torch.cuda.synchronize(); torch.cuda.profiler.start()
            eng.decode_loop(t, 1)
            torch.cuda.synchronize(); torch.cuda.profiler.stop()
    elif mode == "experts":
        # BASELINE config 2's routed-expert matmuls alone (hidden 2048, FFN 512, 256 experts, top-8, Zipf routing) at n tokens
        H, ff, E, K = 2048, 512, 256, 8
        def blocks(n_out, n_in):
            nb = E * n_out * n_in // 64
            b = np.zeros((nb, 36), np.uint8)
            b[:, :4] = rng.integers(0x20, 0x50, (nb, 4)); b[:, 4:] = rng.integers(0, 256, (nb, 32))
            return b.reshape(-1), ((rng.random(E).astype(np.float32) + 0.5) * 0.3)
        (gb, gs), (ub, us), (db, ds) = blocks(ff, H), blocks(ff, H), blocks(H, ff)
        G, U, D = host.Experts(gb, host.NVFP4, H, ff, E, gs), host.Experts(ub, host.NVFP4, H, ff, E, us), host.Experts(db, host.NVFP4, ff, H, E, ds)
        base = (-1.1 * np.log(np.arange(1, E + 1))).astype(np.float32)
        x = rng.standard_normal(n * H).astype(np.float32)
        lg = np.concatenate([base[rng.permutation(E)] for _ in range(n)]).astype(np.float32).reshape(n, E)
        pe = np.exp(lg - lg.max(1, keepdims=True)); probs = (pe / pe.sum(1, keepdims=True)).astype(np.float32).reshape(-1)
        h = np.zeros(n * K * ff, np.float32); scratch = np.zeros_like(h); o = np.zeros(n * K * H, np.float32)
        ops.begin_pass(n)
        route = ops.route(probs, E, K)
        for _ in range(2):
            ops.moe_glu(G, U, route, x, h, scratch); ops.matmul_experts(D, route, h, o)
        ops.check(); torch.cuda.synchronize(); torch.cuda.profiler.start()
        t0 = time.perf_counter()
        ops.moe_glu(G, U, route, x, h, scratch); ops.matmul_experts(D, route, h, o)
        torch.cuda.synchronize(); torch.cuda.profiler.stop()
        print(f"experts {n}: {(time.perf_counter() - t0) * 1e3:.3f} ms (host clock)", file=sys.stderr)
        ops.check(); ops.close()
        return
    else:
        raise SystemExit("--probe: decode:N | prefill:N | step:N | timeline:N | experts:N")
    print(f"{mode} {n}: {eng.last_ms():.3f} ms", file=sys.stderr)
    eng.close(); model.close(); ops.close()


TIMELINE_KERNELS = {2: "k_in_proj", 3: "k_gdn_core", 4: "k_out_proj", 5: "k_attn_prep", 8: "k_moe_glu", 9: "k_moe_down",
                    # stages of the one-kernel step: marks 0 start, 1 end of the stage's work, 2 past the grid barrier
                    17: "mega:embed", 18: "mega:rows", 19: "mega:gdn", 20: "mega:out", 21: "mega:attn_prep", 22: "mega:attn_part",
                    23: "mega:attn_comb", 24: "mega:glu", 25: "mega:down", 26: "mega:advance"}


def print_timeline(eng, dims, tok):
    """itb_timeline_arm / itb_timeline_read around one step: per structured launch, the time from one phase mark to the next
    on block 0 (us), and from the previous launch's last mark to this one's first mark after its dependency wait (the gap)."""
    import collections
    L = eng.L
    L.itb_timeline_read.restype = C.c_long
    slots = 8 * dims["n_layer"] + 8
    assert L.itb_timeline_arm(eng.h, slots) == 0
    eng.decode_loop(tok, 1)
    words = np.zeros(slots * 16, np.uint64)
    L.itb_timeline_read(eng.h, C.c_void_p(words.ctypes.data), slots)
    L.itb_timeline_arm(eng.h, 0)
    agg = collections.OrderedDict()
    prev_last = None
    for w in words.reshape(slots, 16):
        marks = {i: int(v) >> 8 for i, v in enumerate(w) if v}
        if not marks:
            continue
        name = TIMELINE_KERNELS.get(int(w[w != 0][0]) & 255, "?")
        if name.startswith("mega:"):
            # the one-kernel step: intervals against mark 0 (consumers enter the stage); 7/8: the producer reaches the stage's first
            # chunk / has a free slot for it (negative: it ran ahead); 5/6: consumers start / end waiting for that chunk
            for i in sorted(marks):
                if 0 < i < 9:
                    agg.setdefault((name, f"mark {i} - mark 0"), []).append((marks[i] - marks[0]) / 1e3)
                elif i >= 9:   # raw values: 9 = ns thread 0 waited for ring chunks, 10 = ns it worked on them, 11 = chunks
                    agg.setdefault((name, {9: "chunk wait us", 10: "chunk work us", 11: "chunks x1000"}[i]), []).append(marks[i] / 1e3)
            continue
        order = sorted(marks.items(), key=lambda x: x[1])
        for (i, a), (j, b) in zip(order, order[1:]):
            agg.setdefault((name, f"phase {i}->{j}"), []).append((b - a) / 1e3)
        if prev_last is not None and 1 in marks:
            agg.setdefault((name, "gap before"), []).append((marks[1] - prev_last) / 1e3)
        prev_last = max(marks.values())
    for (name, what), v in sorted(agg.items()):
        print(f"{name:12s} {what:14s} n={len(v):3d} mean {np.mean(v):6.2f} us  min {np.min(v):6.2f}  max {np.max(v):6.2f}", file=sys.stderr)


_JSON_FD = None


def emit(obj):
    """The run's one JSON line, on the process's real stdout."""
    data = (json.dumps(obj) + "\n").encode()
    os.write(_JSON_FD if _JSON_FD is not None else 1, data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="product")
    ap.add_argument("--exact", type=int, default=1, help="1 (default): every sum in the CPU path's order, results bit-identical to it; 0: tree-summed F32 dots and the tolerance-class many-token kernels")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the prefill and batch-32 measurements")
    ap.add_argument("--prompt", type=int, default=512, help="prompt tokens before the timed decode steps (BASELINE: 512)")
    ap.add_argument("--cpu-budget", type=float, default=12.0)
    ap.add_argument("--model", default="m35b", choices=["m35b", "l177b"], help="m35b: the headline 35B-A3B shape; l177b: BASELINE config 5's ~177B shape")
    ap.add_argument("--opts", default="", help="extra backend options for --probe runs, e.g. experts=fp4tc")
    ap.add_argument("--probe", default="", help="profiler aid, prints no bench line: 'decode:N' one batched decode step of N sequences, 'prefill:N' one pass of "
                    "N prompt rows, 'step:N' one fused one-token step at N positions, each inside a CUDA profiler range (ncu --profile-from-start off); "
                    "'timeline:N' the per-stage timeline of one step at N positions. Use with --layers.")
    ap.add_argument("--probe-steps", type=int, default=1, help="profiling aid: decode steps inside a 'decode:N' probe's timed region")
    ap.add_argument("--probe-ctx", type=int, default=2048, help="profiling aid: context length of a 'decode:N' probe's engine")
    ap.add_argument("--probe-prompt", type=int, default=64, help="profiling aid: prompt tokens per sequence before a 'decode:N' probe's step")
    ap.add_argument("--layers", type=int, default=0, help="profiling aid: the same shape with fewer layers (small device footprint for ncu captures)")
    args = ap.parse_args()
    # Libraries print banners on stdout (NCCL's version line, for one); stdout must carry the JSON line alone, so everything
    # else written to file descriptor 1 during the run goes to stderr.
    global _JSON_FD
    sys.stdout.flush()
    _JSON_FD = os.dup(1)
    os.dup2(2, 1)
    global PROMPT
    PROMPT = args.prompt
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.probe:
        run_probe(args)
    elif args.impl == "reference":
        args.steps = min(args.steps, 256)   # a CPU step is a whole 2.8 GB token: keep the run within minutes
        run_reference(args, rank, world)
    else:
        run_product(args, rank, world)


if __name__ == "__main__":
    main()
