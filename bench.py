#!/usr/bin/env python
"""Benchmark of the beam-search decoding path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one full decode (encoder, step loop, finalisation) of one batch of synthetic
sentences of the reference decode configuration: 4-layer 1000-unit LSTM encoder/decoder,
30k/30k vocabularies, local-p 'general' attention with feed-input, beam 12, 64 sentences of
10..50 words, T = floor(1.5 S) + 10 expansions, fp32 weights uniform[-0.08, 0.08] (seed 1).
With N > 1 every rank decodes its own batch of the same distribution on its own replica
(weak scaling, no collective in the data path).  Prints ONE JSON line on rank 0.
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
sys.path.insert(0, ROOT)

from linmt_b200 import synth  # noqa: E402

METRIC = "decoded target tokens/sec, beam 12, 4x1000 LSTM"
UNIT = "tokens/s"
FALLBACK_TFLOPS = 1590.0  # used only if MEASURED_PEAKS.json is absent
# DRAM bytes of one launch at 768 rows from ncu captures (see profiles/): read + write
VOCAB_GEMM_TRAFFIC_BYTES = 185.7e6  # 131.1 MB + 54.6 MB, profiles/vocab_gemm_tensor_path_C2.md (algorithmic 218 MB; logits partly still in L2)
# gate GEMM: 66.7 MB measured at K = 3072 (profiles/gate_gemm_tensor_path_C2.md, algorithmic 69.1 MB); the four
# launches of a stack now all run K = 2048 (algorithmic 49.2 MB, scaled from that capture), the first of them reading
# 12.6 MB of input-term table rows besides: average of the four
GATE_GEMM_TRAFFIC_BYTES = 66.7e6 * 49.2 / 69.1 + 12.6e6 / 4


WORKLOADS = {
    # name: (per-rank batch size, scaling, description)
    "C1": (8, "weak", "C1: 2x128 LSTM enc/dec, 1k/1k vocab, greedy, 8 sentences, S in [5,20], T=2S, fp32"),
    "C2": (64, "weak", "C2: 4x1000 LSTM enc/dec, 30k/30k vocab, local-p general attention + feed-input, beam 12, "
                       "64 sentences/batch, S in [10,50], T=floor(1.5S)+10, lp_alpha 0.65, fp32 weights"),
    "C3": (128, "strong", "C3: C2's model in bf16 (fp32 accumulate), beam 12, 4096 sentences, S in [10,80], "
                          "length-bucketed batches of 128 sharded over the GPUs"),
    "C4": (128, "strong", "C4: 4x1024 LSTM, 80k/80k vocab, global dot attention + feed-input, bf16, beam 5, "
                          "1024 sentences, S in [20,100], batches of 128 sharded over the GPUs"),
    "C5": (64, "strong", "C5: ensemble of 4 models (seeds 10-13) of C2's shape, probabilities averaged (reference rule), "
                         "beam 12, 512 sentences, S in [10,60], batches of 64 sharded over the GPUs"),
}


def workload(name: str, rank: int, world: int, precision=None):
    """Returns (config, list of per-rank batches).  C1/C2 are weak-scaled (every rank decodes its
    own batch of the named distribution); C3-C5 are the named fixed jobs, length-bucketed and
    dealt to the ranks (strong scaling)."""
    from linmt_b200 import shard
    c = synth.configs()[name]
    if precision:
        c.precision = precision
    batch, scaling, _ = WORKLOADS[name]
    if scaling == "weak":
        sents = synth.make_sentences(c.n_sent, c.len_lo, c.len_hi, c.desc.Vs, c.zipf_s, c.seeds[0] + 7919 * rank, c.step_rule)
        return c, [sents]
    allsents = c.sentences()
    mine = shard.partition(allsents, world, batch)[rank]
    sub = allsents.subset(mine)
    batches = [sub.subset(b) for b in shard.batches_by_length(sub, batch)]
    return c, batches


def clocks_start():
    q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
    try:
        p = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100"],
                             stdout=f, stderr=subprocess.DEVNULL)
    except OSError:
        return None, f.name
    return p, f.name


def clocks_stop(p, path, device_index: int):
    if p is not None:
        p.terminate()
        try:
            p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            p.kill()
    sm, mx, reasons = [], [], set()
    try:
        for line in open(path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9 or not f[0].isdigit() or int(f[0]) != device_index:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(path)
    except OSError:
        pass
    if not sm:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
    return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(p["bf16_tflops_sustained"]), "measured (cuBLAS bf16, sustained)"
    except Exception:
        return FALLBACK_TFLOPS, "fallback"


def host_threads() -> int:
    """Threads the CPU legs use: every core this process may run on (launchers such as torchrun
    set OMP_NUM_THREADS=1, which would otherwise serialise the CPU port)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def emitted_tokens(out_len: np.ndarray) -> int:
    return int(np.maximum(out_len[:, 0] - 2, 0).sum())


def cpu_leg(c, blobs, sents, n_sample: int, threads: int = 0, repeat: int = 1, ensemble="prob_mean"):
    """Times the CPU checker (a port of the reference's math; the reference has no CPU path
    of its own) on the first n_sample sentences of the batch."""
    from oracle import oracle_py
    sub = sents.subset(range(min(n_sample, sents.n)))
    best = None
    for _ in range(repeat):
        t0 = time.perf_counter()
        o = oracle_py.decode(c.desc, blobs, sub, beam=c.beam, nbest=1, lp_alpha=c.lp_alpha, cp_beta=c.cp_beta,
                             attention=c.attention, precision=c.precision, ensemble=ensemble,
                             threads=threads or host_threads())
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    toks = emitted_tokens(o["len"])
    return toks / best, best, sub.n, threads or host_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    c, batches = workload(args.workload, 0, 1)
    sents = batches[0]
    blob = c.blobs()[0]
    n_sample = 8
    times = []
    toks = 0
    from oracle import oracle_py
    sub = sents.subset(range(n_sample))
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        o = oracle_py.decode(c.desc, [blob], sub, beam=c.beam, nbest=1, lp_alpha=c.lp_alpha, cp_beta=c.cp_beta,
                             threads=host_threads())
        dt = time.perf_counter() - t0
        if i >= args.warmup:
            times.append(dt)
            toks = emitted_tokens(o["len"])
        if sum(times) > 150:
            break
    steps_done = len(times)
    ms = 1e3 * sum(times) / steps_done
    value = toks / (ms / 1e3)
    cores = host_threads()
    sample = f"first {n_sample} of the 64 sentences of the batch per step, rows = {n_sample}*12, all host threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps_done,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config_block(c, sents, args.gpus, args.workload),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference has no CPU forward path and cannot be built here (Boost, GPU-only math); this arm "
                "times the CPU port of its math (oracle/) on the host cores",
    }
    print(json.dumps(line))


def config_block(c, sents, n_gpus, name="C2", n_batches=1, n_sent=None, positions=None):
    return {"workload": WORKLOADS[name][2],
            "sentences_per_step_per_gpu": int(n_sent if n_sent is not None else sents.n), "beam": c.beam,
            "batches_per_step_per_gpu": n_batches,
            "decoder_positions_per_step_per_gpu": int(positions if positions is not None else (sents.steps + 1).sum()),
            "l2": "inputs larger than L2 (>= 0.65 GB of weights streamed every decoder step)",
            "parallelism": f"replicas x{n_gpus}, sentence-sharded, no data-path collective"}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from linmt_b200 import decoder

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    name = args.workload
    c, batches = workload(name, rank, world, args.precision)
    blobs = c.blobs()
    max_src = max(int(b.lengths().max()) for b in batches)
    Tm = max(int(b.steps.max()) for b in batches)
    max_len = Tm + 2
    bmax = max(b.n for b in batches)
    ensemble = c.extra.get("ensemble", "prob_mean")
    dec = decoder.Decoder(c.desc, blobs, beam=c.beam, nbest=1, lp_alpha=c.lp_alpha, cp_beta=c.cp_beta,
                          attention=c.attention, precision=c.precision, ensemble=ensemble,
                          gemm_path=args.gemm_path, max_batch=bmax, max_src_len=max(max_src, 64),
                          max_steps=max(Tm, 100), device=local)
    dev = torch.device("cuda", local)
    dbuf = []
    for b in batches:
        dbuf.append((torch.from_numpy(b.ids.astype(np.int32)).to(dev),
                     torch.zeros((b.n, 1, max_len), dtype=torch.int32, device=dev),
                     torch.zeros((b.n, 1), dtype=torch.int32, device=dev),
                     torch.zeros((b.n, 1), dtype=torch.float32, device=dev)))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    rec = {"ms": 0.0, "n": 0, "flops": 0.0}   # decoder LSTM-stack GEMMs while kernel timing is on

    def step_device():
        """One pass over this rank's batches, ids and outputs resident in HBM."""
        ms = gms = 0.0
        gn = 0
        for b, (d_ids, d_tok, d_len, d_score) in zip(batches, dbuf):
            dec.decode_device(d_ids.data_ptr(), b.off, b.steps, max_len, d_tok.data_ptr(), d_len.data_ptr(), d_score.data_ptr())
            st = dec.stats()
            ms += st["last_decode_ms"]; gms += st["last_gemm_ms"]; gn += st["last_gemm_launches"]
            rec["ms"] += st["last_rec_gemm_ms"]; rec["n"] += st["last_rec_gemm_launches"]; rec["flops"] += st["last_rec_gemm_flops"]
        return ms, gms, gn

    # ---- device-resident leg: `value` (no per-kernel events inside: they cost ~4 % and end the
    # overlap of consecutive kernels at every event) ----
    for _ in range(args.warmup):
        step_device()
    s0 = dec.stats()
    barrier()
    clk_p, clk_path = clocks_start() if rank == 0 else (None, None)
    dev_ms = 0.0
    w0 = time.perf_counter()
    for _ in range(args.steps):
        a, _, _ = step_device()
        dev_ms += a
    barrier()
    wall_ms = 1e3 * (time.perf_counter() - w0)
    s1 = dec.stats()
    launches = s1["kernel_launches"] - s0["kernel_launches"]
    toks = sum(emitted_tokens(d[2].cpu().numpy()) for d in dbuf)
    row_steps = s1["decoder_row_steps"] - s0["decoder_row_steps"]

    # ---- the same steps once more with CUDA events around every vocabulary GEMM and every
    # decoder LSTM stack: the roofline figures (clock sampling runs on over this pass) ----
    dec.set_kernel_timing(True)
    rec.update(ms=0.0, n=0, flops=0.0)
    gemm_ms, gemm_n, timed_ms = 0.0, 0, 0.0
    for _ in range(args.steps):
        a, g, n = step_device()
        timed_ms += a; gemm_ms += g; gemm_n += n
    barrier()
    dec.set_kernel_timing(False)
    clocks = clocks_stop(clk_p, clk_path, local) if rank == 0 else None

    # ---- end-to-end leg through the public host API: pinned host buffers, copies inside ----
    hbatches, pins = [], []
    for b in batches:
        h_ids = torch.from_numpy(b.ids.astype(np.int32)).pin_memory()
        pins.append(h_ids)
        hbatches.append(synth.Sentences(h_ids.numpy(), b.off, b.steps))
    outs = None
    for _ in range(min(args.warmup, 2)):
        outs = [dec.decode(hb) for hb in hbatches]
    barrier()
    e0 = time.perf_counter()
    for _ in range(args.steps):
        outs = [dec.decode(hb) for hb in hbatches]
    barrier()
    e2e_wall_ms = 1e3 * (time.perf_counter() - e0)
    e_toks = sum(emitted_tokens(o["len"]) for o in outs)
    h2d = int(sum(b.ids.nbytes + 4 * 4 * b.n for b in batches))
    d2h = int(sum(o["tok"].nbytes + o["len"].nbytes + o["score"].nbytes + o["vit"].nbytes for o in outs))

    # ---- reduce over ranks: max time, summed tokens ----
    vals = torch.tensor([dev_ms, wall_ms, e2e_wall_ms, gemm_ms], dtype=torch.float64, device=dev)
    n_sent_local = sum(b.n for b in batches)
    positions_local = int(sum(int((b.steps + 1).sum()) for b in batches))
    sums = torch.tensor([toks, e_toks, launches, row_steps, gemm_n, n_sent_local], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    dev_ms_local = dev_ms
    dev_ms, wall_ms, e2e_wall_ms, gemm_ms_max = vals.tolist()
    toks_all, e_toks_all, launches_all, row_steps_all, gemm_n_all, n_sent_all = sums.tolist()

    if rank == 0:
        ms_per_step = dev_ms / args.steps
        value = toks_all * args.steps / (dev_ms / 1e3)
        e2e_value = e_toks_all * args.steps / (e2e_wall_ms / 1e3)
        # roofline of the dominant kernel (the vocabulary GEMM): algorithmic FLOPs = 2 * rows * H * V per member
        H, V = c.desc.H, c.desc.V
        flops_local = 2.0 * (s1["decoder_row_steps"] - s0["decoder_row_steps"]) * H * V * len(blobs)
        peak, peak_src = peaks()
        tensor = args.gemm_path != "simt"
        fp32 = c.precision != "bf16"

        def roof(kernel, flops, ms, n, products, traffic):
            """Roofline block of one GEMM class: algorithmic flops over the CUDA-event time of its launches."""
            ach = flops / (ms / 1e3) / 1e12 if ms > 0 else None
            return {"bound": "tensor", "kernel": kernel, "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                    "frac": (ach / peak) if ach else None, "traffic": traffic, "peak_source": peak_src,
                    "launches": int(n), "avg_launch_ms": ms / max(n, 1), "share_of_step": ms / timed_ms if timed_ms else None,
                    "bf16_products_per_product": products if tensor else 0,
                    "tensor_pipe_tflops": ach * products if (ach and tensor) else None,
                    "tensor_pipe_frac": ach * products / peak if (ach and tensor) else None,
                    "note": "launch durations by CUDA events in a second pass over the same steps (the timed pass for `value` carries no per-kernel events); achieved = algorithmic fp32 flops; on the fp32 tensor path every product is computed as "
                            "this many bf16 partial products (operands split into bf16 planes), which is what "
                            "tensor_pipe_* counts; the bf16 path runs 1"}

        r_voc = roof("vocabulary GEMM [rows,H]x[H,V] (" + args.gemm_path + " path; the default computes it as one fp16 product and recomputes the top candidates in the softmax kernel)", flops_local, gemm_ms, gemm_n,
                     (4 if args.gemm_path in ("tensor2", "tensor3") else (1 if args.gemm_path in ("tensor_v16", "tensor_v16x", "auto") and len(blobs) == 1 else 3)) if fp32 else 1, VOCAB_GEMM_TRAFFIC_BYTES if name == "C2" and fp32 and args.gemm_path == "tensor" else None)
        r_rec = roof("decoder LSTM gate GEMMs [rows,2H|3H]x[.,4H], fused cell update (" + args.gemm_path + " path)",
                     rec["flops"], rec["ms"], rec["n"],
                     {"tensor2": 4, "tensor3": 6}.get(args.gemm_path, 3) if fp32 else 1,
                     GATE_GEMM_TRAFFIC_BYTES if name == "C2" and fp32 and args.gemm_path in ("auto", "tensor") else None)
        dominant, other = (r_rec, r_voc) if rec["ms"] >= gemm_ms else (r_voc, r_rec)
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            v, secs, ns, cores = cpu_leg(c, blobs, batches[0], 16, ensemble=ensemble)
            cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                   "sample": f"first {ns} sentences of the first batch, batched (rows = {ns}*{c.beam}), {secs:.1f} s of CPU work"}
        scaling = WORKLOADS[name][1]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "bf16" if c.precision == "bf16" else "f32", "data": "synthetic",
            "config": config_block(c, batches[0], world, name, len(batches), n_sent_local, positions_local),
            "positions_per_s": row_steps_all / c.beam / (dev_ms / 1e3),
            "sentences_per_step": int(n_sent_all),
            "wall_ms_per_step": wall_ms / args.steps,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_wall_ms / args.steps},
            "gpu_launches": int(launches_all),
            "roofline": dominant, "roofline_other": [other],
            "cpu_baseline": cpu, "clocks": clocks, "gemm_path": args.gemm_path,
        }
        print(json.dumps(line))
    dec.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--gemm-path", default="auto", choices=["auto", "simt", "tensor", "tensor2", "tensor3", "tensor_v16", "tensor_v16x"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="C2", choices=sorted(WORKLOADS))
    ap.add_argument("--precision", default=None, choices=["fp32", "bf16"], help="override the workload's precision")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
