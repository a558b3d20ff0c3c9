"""Benchmark of the GPT-2 decode path on B200 (one process per GPU).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload xl-q4_0-b256|medium-q4_0-b64|small-q8_0-b1|small-f32-b1|xl-q4_0-b1]
                    [--precision bf16x3|bf16|fp32] [--scaling strong|weak]

A "step" is one KV-cached greedy decode step of the whole batch (one new token per sequence).
Default workload: GPT-2 XL, Q4_0 weights, ONE batch of 256 sequences, 512-token prompts, 256 decoded
tokens, fp32 KV cache.  Sequences are independent, so the batch is sharded over the N GPUs (256 / N
each) with replicated weights and no collective on the data path (`--scaling strong`, the default);
`--scaling weak` instead keeps the workload's whole batch on every GPU (global batch = batch x N).
The timed steps are centred on the middle of the decode phase (context = prompt + decode / 2), so
`value` is the configuration's average step, and the CPU arm is timed at the same contexts.
Prints ONE JSON line on rank 0.

* ``value``  decode tokens/s with token ids resident in HBM (CUDA events on the library's stream,
             barrier + synchronize on both sides, max over ranks).
* ``e2e``    the same steps through ``GPT2.forward`` (the call of apps/gpt2/gpt2.lisp:104): host
             ids in (pinned H2D) and host ids out (D2H) inside every timed step.
* ``roofline``  attention-decode kernel (the dominant one: the KV cache is re-read every step),
             algorithmic bytes = 2 * t * d_model * 4 B per sequence per layer, timed live with
             CUDA events around its launches inside the timed region.
* ``cpu_baseline``  the CPU oracle (restatement of BACKEND=CLANG's arithmetic, one thread as the
             reference runs) on a bounded sample; ``--impl reference`` times the same code with
             every host thread.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (model, weight type, total batch, prompt length, decode length)
    "xl-q4_0-b256": ("gpt2-xl", "q4_0", 256, 512, 256),
    "medium-q4_0-b64": ("gpt2-medium", "q4_0", 64, 128, 128),
    "small-q8_0-b1": ("gpt2", "q8_0", 1, 128, 256),
    "small-f32-b1": ("gpt2", "f32", 1, 16, 100),
    "xl-q4_0-b1": ("gpt2-xl", "q4_0", 1, 512, 256),   # one sequence: every linear is a dequant-GEMV
}
METRIC = "gpt2_decode_tokens_per_s"
BPW = {"f32": 4.0, "q8_0": 34 / 32, "q4_0": 18 / 32}


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return 6650.0, "fallback (no MEASURED_PEAKS.json beside bench.py)"


def load_tensor_peak():
    """(burst, sustained) dense bf16 TFLOP/s of MEASURED_PEAKS.json, else the fallback pair."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            j = json.load(f)
            return float(j["bf16_tflops"]), float(j["bf16_tflops_sustained"])
    except Exception:
        return 1590.0, 1400.0


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(device), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        # the first samples may precede the load; the median of the upper half reflects the timed region
        top = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(top) if top else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def host_cores() -> int:
    """Host threads this process may use: the affinity mask, not OMP_NUM_THREADS (which
    `torch.distributed.run` sets to 1 for every rank)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def dequantised_state_dict(sd):
    """fp32 copies of the packed matrices, as the reference holds its weights (oracle side only)."""
    import oracle as O
    from caten_b200 import synthetic as S
    O.build()
    return {k: (O.dequant(v.ggml_type, v.data, v.rows * v.cols).reshape(v.rows, v.cols) if isinstance(v, S.Packed) else v)
            for k, v in sd.items()}


def cpu_decode_sample(params, fsd, first_context: int, warmup: int, steps: int, threads: int, budget_s: float):
    """Times the CPU oracle on `steps` decode steps of ONE sequence whose first timed step sees
    `first_context` cached tokens (KV cache pre-filled with a value pattern: its contents do not
    change the work), after `warmup` untimed steps."""
    import oracle as O
    need = first_context + steps + 2
    wpe = fsd["wpe.weight"]
    T = min(need, wpe.shape[0])
    steps = max(1, min(steps, T - first_context - 1))
    warmup = max(1, min(warmup, first_context - 1))
    O.set_threads(threads)
    m = O.GPT2(params.n_layers, params.dim, params.n_heads, params.vocab_size, T, 1, {**fsd, "wpe.weight": wpe[:T]})
    m.fill_cache(0.01)
    ids = np.zeros((1, 1), np.float32)
    for i in range(warmup):  # page in the weights, warm the caches
        m.step(ids, first_context - warmup + i, want_logits=False)
    done, t0 = 0, time.perf_counter()
    for i in range(steps):
        out, _ = m.step(ids, first_context + i, want_logits=False)
        ids = out.reshape(1, 1).astype(np.float32)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    m.close()
    O.set_threads(1)
    return done / dt, done, dt


def oracle_parity(model, params, fsd, nb: int, precision: str, threads: int, prompt_len: int = 16, steps: int = 3):
    """A short run of the benchmarked model object (same weights, batch, precision, kernels and
    CUDA-graph path) against the strict-fp32 CPU oracle: the first one or two sequences are
    compared, teacher-forced on the oracle's ids, logits within the tolerance of the precision."""
    import oracle as O
    from caten_b200 import synthetic as S
    nchk = min(2, nb)
    T = prompt_len + steps + 1
    prompts = S.synth_prompts(nb, prompt_len, params.vocab_size, seed=7)
    O.set_threads(threads)
    ref = O.GPT2(params.n_layers, params.dim, params.n_heads, params.vocab_size, T, nchk, {**fsd, "wpe.weight": fsd["wpe.weight"][:T]})
    tokens, pos = prompts.copy(), 0
    worst_abs, worst_rel, ids_equal, ids_checked = 0.0, 0.0, 0, 0
    for _ in range(1 + steps):
        ids_ref, lg_ref = ref.step(tokens[:nchk, pos:], pos)
        ids = model.forward(tokens[:, pos:], tokens.shape[1] - pos, pos)
        lg = model.logits()[:nchk]
        err = float(np.abs(lg - lg_ref).max())
        worst_abs = max(worst_abs, err)
        worst_rel = max(worst_rel, err / float(np.abs(lg_ref).max()))
        top2 = np.sort(lg_ref, axis=1)[:, -2:]
        decisive = (top2[:, 1] - top2[:, 0]) > 20.0 * err + 1e-6
        ids_equal += int((ids[:nchk][decisive] == ids_ref[decisive]).sum())
        ids_checked += int(decisive.sum())
        nxt = ids.copy()
        nxt[:nchk] = ids_ref          # teacher forcing on the checked sequences
        pos = tokens.shape[1]
        tokens = np.concatenate([tokens, nxt.reshape(-1, 1)], axis=1)
    ref.close()
    O.set_threads(1)
    ok = (worst_rel <= 2e-2) if precision == "bf16" else (worst_abs <= 1e-3)
    ok = ok and ids_equal == ids_checked
    return {"ok": bool(ok), "against": "CPU oracle, strict fp32", "sequences": nchk, "prompt": prompt_len, "decode_steps": steps,
            "logits_max_abs_err": worst_abs, "logits_max_rel_err": worst_rel,
            "tolerance": "relative 2e-2" if precision == "bf16" else "max-abs 1e-3",
            "ids_equal_where_decisive": f"{ids_equal}/{ids_checked}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="xl-q4_0-b256", choices=sorted(WORKLOADS))
    ap.add_argument("--precision", default="bf16x3", choices=["fp32", "bf16", "bf16x3"])
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"], help="replay decode steps from a CUDA graph (auto = on; off launches kernel by kernel)")
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="strong: one batch of the workload's size split over the GPUs; weak: that batch on every GPU")
    ap.add_argument("--dist-plane", default="capi", choices=["capi", "torch"],
                    help="who moves the weights and the ids between GPUs: the library's own NCCL entry points "
                         "(caten_b200_dist_*, what a Lisp host would call) or torch.distributed")
    ap.add_argument("--batch", type=int, default=None,
                    help="override the workload's total batch (e.g. 32 = what one of 8 GPUs holds in a strong-scaled xl-q4_0-b256 run); "
                         "the batch that ran is the one config.workload names")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the short oracle check of the benchmarked model")
    ap.add_argument("--no-extras", action="store_true", help="skip the prefill/GEMV/kernel-breakdown side measurements")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    model_name, wtype, batch, prompt_len, decode_len = WORKLOADS[args.workload]
    if args.batch is not None:
        if args.batch < 1:
            raise SystemExit("--batch must be at least 1")
        batch = args.batch
    if args.scaling == "weak":
        batch *= world   # global batch; every rank keeps the workload's own batch
    W = max(0, args.warmup)
    K = args.steps if args.steps is not None else max(1, min(64, decode_len - W - 1))
    if W + K > decode_len:
        K = max(1, decode_len - W)
    # untimed steps after the prompt that bring the cache to the middle of the decode phase
    A = max(0, min(decode_len // 2 - K // 2 - W, decode_len - W - K))
    T = prompt_len + decode_len
    first_timed_context = prompt_len + A + W    # tokens already cached when the first timed step starts

    from caten_b200 import synthetic as S
    params = S.GPT2_SIZES[model_name]
    # identical in both arms: what is computed, not how
    config = {"workload": f"{model_name} {wtype} batch {batch} prompt {prompt_len} decode {decode_len}",
              "model_dims": f"L{params.n_layers} d{params.dim} H{params.n_heads} V{params.vocab_size}",
              "kv_cache": f"fp32 [B,H,{T},64] per layer", "weights_seed": 0, "prompt_seed": 0,
              "timed_context_tokens": [first_timed_context + 1, first_timed_context + K],
              "l2": "inputs larger than L2: every step re-reads the KV cache and all weights"}

    # ------------------------------------------------------------------ reference arm (CPU)
    if args.impl == "reference":
        if rank != 0:
            return
        sd = S.synth_state_dict(params, wtype, seed=0, max_seq_len=T)
        threads = host_cores()
        fsd = dequantised_state_dict(sd)
        tps, done, dt = cpu_decode_sample(params, fsd, first_timed_context, W, K, threads, budget_s=150.0)
        sample = (f"{done} decode steps of 1 of the {batch} sequences at contexts {first_timed_context + 1}..{first_timed_context + done}, "
                  f"KV cache pre-filled, {threads} threads (OpenMP over output rows and heads)")
        line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": done, "warmup": W,
                "ms_per_step": 1000.0 * dt / done, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config,
                "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
                "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    # ------------------------------------------------------------------ B200 arm
    import torch
    import torch.distributed as dist
    from caten_b200 import dist as D
    from caten_b200.gpt2 import GPT2
    from caten_b200.runtime import B200Runtime

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    b0, nb = D.shard_batch(batch, world, rank)
    if nb < 1:
        raise SystemExit("more ranks than sequences")

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    rt = B200Runtime(local_rank)
    sd = S.synth_state_dict(params, wtype, seed=0, max_seq_len=T) if rank == 0 else None
    def exchange(obj):   # rank 0's small host object on every rank (control plane: the launcher's store)
        box = [obj]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    if world > 1 and args.dist_plane == "capi":
        D.capi_group_init(rt, rank, world, exchange)
        arena, index = D.capi_broadcast_state_dict(rt, sd, rank, exchange)   # ncclBroadcast of the packed weights at load
        stubs, ptrs = D.arena_views(arena.ptr, index)
        model = GPT2(rt, params, stubs, max_seq_len=T, batch=nb, precision=args.precision, device_blobs=ptrs)
        rt.sync()
        arena.close()
    elif world > 1:
        arena, index = D.broadcast_state_dict(sd, dev)   # NCCL broadcast of the packed weights at load
        stubs, ptrs = D.device_views(arena, index)
        torch.cuda.synchronize()
        model = GPT2(rt, params, stubs, max_seq_len=T, batch=nb, precision=args.precision, device_blobs=ptrs)
        rt.sync()
        del arena
    else:
        model = GPT2(rt, params, sd, max_seq_len=T, batch=nb, precision=args.precision)
    prompts = S.synth_prompts(batch, prompt_len, params.vocab_size, seed=0)[b0:b0 + nb]
    ext = torch.cuda.ExternalStream(rt.stream, device=dev)

    def ev():
        e = torch.cuda.Event(enable_timing=True)
        e.record(ext)
        return e

    # ---- prefill (fills the cache; timed on the side)
    ids_dev = rt.transfer_from_array(prompts.astype(np.float32))
    a = model._dev_ids.view(0, (nb, 1))
    b = model._dev_ids.view(nb, (nb, 1))
    first = rt.open_buffer((nb,), np.int64)
    rt.sync(); barrier()
    e0 = ev()
    model.forward_device(ids_dev, prompt_len, 0, first)
    e1 = ev()
    rt.sync()
    prefill_ms = max_over_ranks(e0.elapsed_time(e1))
    first_ids = first.numpy()

    def run_device_steps(n_start, count, cur, nxt, hist=None, h0=0):
        for i in range(count):
            model.forward_device(cur, 1, n_start + i, nxt)
            if hist is not None:
                rt.lib.caten_b200_d2d(rt.ctx, hist.ptr + (h0 + i) * nb * 8, nxt.ptr, nb * 8)
            cur, nxt = nxt, cur
        return cur, nxt

    # ---- timed region 1: device-resident decode
    # graph mode: one C call per token replaying a captured CUDA graph (what a serving loop uses when
    # the per-GPU batch is small and kernel launches would otherwise pace the step); eager mode:
    # one launch per kernel, which lets CUDA events bracket the attention kernel inside the region.
    # Untimed first: A steps that advance the cache to mid-decode, then W warm-up steps.
    use_graph = args.graph != "off"
    pre = A + W
    hist = rt.open_buffer((pre + K, nb), np.int64)   # row i = ids produced by the step at position prompt_len + i
    first_dev = rt.transfer_from_array(first_ids)
    first_steps = None
    if use_graph:
        model.decode_device_buffers(first_dev, prompt_len, 2, None)   # captures the graph
        done = 0
        if pre >= 2 * W + K and W > 0:
            # side measurement on the way: the first K steps after the prompt (after W warm-up steps), the window
            # earlier records of this benchmark were taken on; the contexts are ~20 % shorter than at mid-decode
            model.decode_device_buffers(first_dev, prompt_len, W, hist)
            rt.sync(); barrier()
            f0 = ev()
            model.decode_device_buffers(hist.view((W - 1) * nb, (nb,)), prompt_len + W, K, hist.view(W * nb, (K, nb)))
            f1 = ev()
            rt.sync()
            first_ms = max_over_ranks(f0.elapsed_time(f1))
            first_steps = {"contexts": [prompt_len + W + 1, prompt_len + W + K], "ms_per_step": first_ms / K,
                           "tokens_per_s": batch * K / (first_ms / 1e3)}
            done = W + K
        if pre - done:
            src = hist.view((done - 1) * nb, (nb,)) if done else first_dev
            model.decode_device_buffers(src, prompt_len + done, pre - done, hist.view(done * nb, (pre - done, nb)))
        cur = hist.view((pre - 1) * nb, (nb,)) if pre else first_dev
    else:
        rt.lib.caten_b200_h2d(rt.ctx, a.ptr, first_ids.ctypes.data, first_ids.nbytes)
        cur, nxt = run_device_steps(prompt_len, pre, a, b, hist, 0)
    rt.sync(); barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = model.launch_count
    if not use_graph:
        rt.profile_begin(["attn_decode"])
    torch.cuda.synchronize(); barrier()
    e0 = ev()
    if use_graph:
        model.decode_device_buffers(cur, first_timed_context, K, hist.view(pre * nb, (K, nb)))
    else:
        cur, nxt = run_device_steps(first_timed_context, K, cur, nxt, hist, pre)
    e1 = ev()
    rt.sync(); torch.cuda.synchronize(); barrier()
    dec_ms = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if sampler else None
    launches = model.launch_count - launches0
    ids_device_path = hist.numpy()
    value = batch * K / (dec_ms / 1e3)
    if use_graph:
        # launches inside a graph cannot be bracketed: time the attention kernel in an eager replay
        # of the same steps (same inputs, same positions) right after the timed region
        rt.profile_begin(["attn_decode"])
        model.decode_device_buffers(cur, first_timed_context, K, None)
    prof = rt.profile_end()

    # roofline of the attention-decode kernel: average context over the timed steps
    attn_ms, attn_calls = prof.get("attn_decode", (0.0, 0))
    t_mean = first_timed_context + (K - 1) / 2.0 + 1       # keys read per step incl. the new one
    attn_bytes = nb * 2 * t_mean * params.dim * 4.0        # per launch (one layer), K and V rows once
    peak, peak_src = load_peaks()
    attn_avg_s = (attn_ms / attn_calls / 1e3) if attn_calls else float("nan")
    achieved = attn_bytes / attn_avg_s / 1e9 if attn_calls else None
    roofline = {"bound": "hbm", "kernel": "attn_decode_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": (achieved / peak) if achieved else None,
                # DRAM bytes per launch: ncu measured dram read+write = 1.008 x algorithmic on a 64-sequence launch of
                # this kernel (profiles/attn_decode_kernel_b64_h25_t701.md); traffic grows with sequences x context
                "traffic": attn_bytes * 1.008, "traffic_source": "ncu capture of a smaller launch, scaled by sequences x context",
                "peak_source": peak_src,
                "bytes_per_launch": attn_bytes, "avg_launch_us": attn_avg_s * 1e6, "launches_timed": attn_calls,
                "timed_in": "eager replay of the timed steps (graph mode)" if use_graph else "the timed region",
                "share_of_step": (attn_ms / (dec_ms)) if dec_ms else None}
    # whole-step algorithmic bytes (weights once + KV read + small terms), for context
    d, Ln, V = params.dim, params.n_layers, params.vocab_size
    p_lin = 12 * d * d * Ln + V * d
    step_bytes = p_lin * BPW[wtype] + 4 * (13 * d * Ln + 2 * d) + nb * (2 * d * 4 + Ln * 2 * t_mean * d * 4 + Ln * 2 * d * 4 + 8)
    step_frac = step_bytes / (dec_ms / K / 1e3) / 1e9 / peak

    # ---- timed region 2: the public host API, host ids in / out every step (same positions)
    tok = (ids_device_path[A - 1] if A else first_ids).reshape(nb, 1)
    for i in range(W):
        tok = model.forward(tok, 1, prompt_len + A + i).reshape(nb, 1)
    rt.sync(); barrier()
    t0 = time.perf_counter()
    e2e_ids = []
    for i in range(K):
        tok = model.forward(tok, 1, first_timed_context + i).reshape(nb, 1)
        e2e_ids.append(tok[:, 0].copy())
    rt.sync(); barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e = {"value": batch * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": nb * 4 * world, "d2h_bytes_per_step": nb * 8 * world,
           "ms_per_step": 1000.0 * e2e_s / K, "timer": "host wall clock between barrier+synchronize pairs, max over ranks"}
    same_ids = bool((np.stack(e2e_ids) == ids_device_path[pre:]).all())

    # gather the generated ids on all ranks (the only collective after load)
    if world > 1:
        if args.dist_plane == "capi":
            gathered = D.capi_gather_ids(rt, ids_device_path, batch, world)
        else:
            gathered = D.gather_ids(torch.from_numpy(ids_device_path).to(dev), batch, world)
        assert tuple(gathered.shape) == (pre + K, batch)
        assert (np.asarray(gathered.cpu() if hasattr(gathered, "cpu") else gathered)[:, b0:b0 + nb] == ids_device_path).all()

    extras = {}
    if not args.no_extras:
        # per-class breakdown of a few decode steps (all classes timed; not part of `value`)
        rt.lib.caten_b200_h2d(rt.ctx, a.ptr, first_ids.ctypes.data, first_ids.nbytes)
        rt.sync()
        rt.profile_begin(None)
        run_device_steps(first_timed_context, min(K, 8), a, b)
        br = rt.profile_end()
        tot = sum(v[0] for v in br.values()) or 1.0
        extras["kernel_ms_share"] = {k: round(v[0] / tot, 4) for k, v in br.items()}
        # prefill: the real one above (the precision of the run), plus one group of sequences (what one pass of the
        # prefill processes at a time) in each tensor-core precision on rank 0, with the useful FLOP rate
        # (2 x 12 d^2 L per token + causal attention 2 s d L per token + the last row's lm_head)
        extras["prefill"] = {"tokens_per_s": sum_over_ranks(nb * prompt_len) / (prefill_ms / 1e3), "ms": prefill_ms,
                             "tokens": batch * prompt_len, "precision": args.precision}
        if rank == 0 and world == 1 and args.precision != "fp32":
            _, bf16_peak = load_tensor_peak()
            gsz = max(1, min(nb, 8192 // prompt_len))
            flop_per_tok = 2.0 * 12 * params.dim ** 2 * params.n_layers + 2.0 * prompt_len * params.dim * params.n_layers
            for prec in ("bf16x3", "bf16"):
                pm = GPT2(rt, params, sd, max_seq_len=prompt_len + 8, batch=gsz, precision=prec)
                pin = rt.transfer_from_array(prompts[:gsz].astype(np.float32))
                pout = rt.open_buffer((gsz,), np.int64)
                pm.forward_device(pin, prompt_len, 0, pout); rt.sync()      # warm-up (allocations, attributes)
                p0 = ev(); pm.forward_device(pin, prompt_len, 0, pout); p1 = ev(); rt.sync()
                ms = p0.elapsed_time(p1)
                tf = flop_per_tok * gsz * prompt_len / (ms / 1e3) / 1e12
                rt.profile_begin(); pm.forward_device(pin, prompt_len, 0, pout); by_class = rt.profile_end()   # a third pass, kernel classes bracketed by events
                extras["prefill"][f"group_{prec}"] = {"sequences": gsz, "tokens": gsz * prompt_len, "ms": ms, "tokens_per_s": gsz * prompt_len / (ms / 1e3),
                                                       "useful_TFLOP/s": tf, "frac_of_sustained_bf16_peak": tf / bf16_peak,
                                                       "issued_frac": tf * (3 if prec == "bf16x3" else 1) / bf16_peak,
                                                       "ms_by_kernel_class": {k: round(v[0], 3) for k, v in by_class.items()}}
                pm.close(); pin.close(); pout.close()
            # configuration 2 of the reference's benchmark list: relu(A[4096x768] . B[768x3072]), fp32 in and out
            A_, B_ = S.synth_relu_gemm(seed=1)
            da, db = rt.transfer_from_array(A_), rt.transfer_from_array(B_)
            from caten_b200 import _lib as L_
            dc = rt.open_buffer((4096, 3072))
            rm = {}
            for prec in ("bf16x3", "bf16", "fp32"):
                pc = L_.PRECISIONS[prec]

                def once():   # straight through the C ABI into a caller-owned output: no allocation inside the timed loop
                    L_.check(rt.ctx, rt.lib.caten_b200_relu_matmul(rt.ctx, da.ptr, db.ptr, dc.ptr, 4096, 768, 3072, pc))
                for _ in range(3):
                    once()
                rt.sync()
                p0 = ev()
                for _ in range(10):
                    once()
                p1 = ev(); rt.sync()
                us = p0.elapsed_time(p1) / 10 * 1e3
                tf = 2.0 * 4096 * 768 * 3072 / (us / 1e6) / 1e12
                rm[prec] = {"us": us, "useful_TFLOP/s": tf, "frac_of_sustained_bf16_peak": tf / bf16_peak}
            extras["relu_matmul_4096x768x3072"] = rm
            da.close(); db.close(); dc.close()
        if rank == 0 and wtype != "f32":
            # dequant-GEMV on the model's own matrices, cycling over all layers so the weights
            # (hundreds of MB in total) do not stay in the 126 MB L2
            x1 = rt.open_buffer((1, 4 * d))
            res = {}
            for kind, rows, cols in (("attn.c_attn", 3 * d, d), ("attn.c_proj", d, d), ("mlp.c_fc", 4 * d, d), ("mlp.c_proj", d, 4 * d)):
                ws = [model.weights[f"h.{l}.{kind}.weight"] for l in range(Ln)]
                y = rt.open_buffer((1, rows))
                xin = x1.view(0, (1, cols))
                for w in ws:
                    rt.linear(w, xin, out=y)
                rt.sync()
                s0 = ev()
                for _ in range(3):
                    for w in ws:
                        rt.linear(w, xin, out=y)
                s1 = ev()
                rt.sync()
                per = s0.elapsed_time(s1) / (3 * len(ws)) / 1e3
                nbytes = ws[0].packed_nbytes
                res[f"{rows}x{cols}"] = {"GB/s": nbytes / per / 1e9, "frac_of_peak": nbytes / per / 1e9 / peak, "us": per * 1e6}
            w = model.weights["lm_head.weight"]
            y = rt.open_buffer((1, V)); xin = x1.view(0, (1, d))
            rt.linear(w, xin, out=y); rt.sync()
            s0 = ev()
            for _ in range(10):
                rt.linear(w, xin, out=y)
            s1 = ev(); rt.sync()
            per = s0.elapsed_time(s1) / 10 / 1e3
            res[f"{V}x{d}"] = {"GB/s": w.packed_nbytes / per / 1e9, "frac_of_peak": w.packed_nbytes / per / 1e9 / peak, "us": per * 1e6,
                               "note": "a 45 MB matrix can stay resident in the 126 MB L2 between launches"}
            extras["dequant_gemv"] = res

    # ---- outside the timed regions, rank 0: oracle check of the benchmarked model, CPU baseline
    cpu, parity = None, None
    need_oracle = rank == 0 and ((not args.no_parity) or (world == 1 and not args.no_cpu_baseline))
    if need_oracle:
        fsd = dequantised_state_dict(sd)
        if not args.no_parity:
            parity = oracle_parity(model, params, fsd, nb, args.precision, host_cores())
        if world == 1 and not args.no_cpu_baseline:
            tps, done, dt = cpu_decode_sample(params, fsd, first_timed_context, 1, 24, 1, budget_s=15.0)   # about 10-15 s of CPU work
            cpu = {"value": tps, "unit": "tokens/s", "cores": 1, "kind": "port",
                   "sample": f"{done} decode steps of 1 of the {batch} sequences at contexts {first_timed_context + 1}..{first_timed_context + done} "
                             f"(KV cache pre-filled), {dt:.1f} s; BACKEND=CLANG executes its kernels on one thread"}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": dec_ms / K, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
                "dtype": "f32 (attention, LayerNorm, accumulation); linears " + {"fp32": "f32", "bf16": "bf16 operands", "bf16x3": "split-bf16 operands (3 products)"}[args.precision] + " on tcgen05",
                "data": "synthetic", "config": config,
                "run": {"parallelism": f"batch-sharded x{world}, weights replicated", "dist_plane": args.dist_plane if world > 1 else None, "global_batch": batch, "local_batch": nb, "precision": args.precision,
                        "cuda_graph": use_graph, "untimed_steps_before": pre, "first_decode_steps": first_steps},
                "roofline": roofline, "whole_step": {"algorithmic_bytes": step_bytes, "frac_of_hbm_peak": step_frac},
                "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
                "parity_checked": bool(parity and parity["ok"]), "parity": parity,
                "ids_host_path_equal_device_path": same_ids, **extras}
        print(json.dumps(line))
    model.close()
    rt.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
