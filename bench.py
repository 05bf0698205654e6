#!/usr/bin/env python
"""Benchmark of the beam-search decoding path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one full decode (encoder, step loop, finalisation) of one batch of synthetic
sentences of the reference decode configuration: 4-layer 1000-unit LSTM encoder/decoder,
30k/30k vocabularies, local-p 'general' attention with feed-input, beam 12, 64 sentences of
10..50 words, T = floor(1.5 S) + 10 expansions, fp32 weights uniform[-0.08, 0.08] (seed 1).
With N > 1 every rank decodes its own batch of the same distribution on its own replica
(weak scaling, no collective in the data path).  Beside that headline the line carries `strong_c3`: the
fixed 4096-sentence bf16 job of the throughput configuration, length-bucketed, dealt to the N ranks and
gathered once (strong scaling), with per-rank work and times.  Prints ONE JSON line on rank 0.
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
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes (read + write) of ONE launch of each kernel class at the full width of the C2 batch (768 rows), from
# ncu captures of this benchmark's own C2 decode (dram__bytes_read.sum + dram__bytes_write.sum of one launch; the
# summaries with the capture commands are committed with the profiles).  None = no capture for that class.
C2_TRAFFIC_BYTES = {
    "lstm_gemm": 43.5e6,        # first layer 45.74 MB (with input-term table rows), the others 42.72 MB
    "vocab_gemm": 77.2e6,       # 63.40 MB read (the weights) + 13.82 MB written (fp16 logits, most of them still in L2)
    "attn_proj_gemm": 15.8e6, "attn_out_gemm": 10.56e6,
    "softmax_topk": 56.0e6,     # the fp16 logits once + candidates' weight rows (cold-cache capture)
    "gather": 10.66e6, "attention": 19.55e6, "beam_select": 0.11e6,
}


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


def workload(name: str, rank: int, world: int, precision=None, n_sentences=None):
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
    allsents = c.sentences(n_sentences)   # None = the configuration's own job size
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
    """(sustained bf16 TFLOP/s, HBM GB/s, where the numbers come from)."""
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(p["bf16_tflops_sustained"]), float(p["hbm_gbs"]), "measured (cuBLAS bf16 sustained; copy bandwidth)"
    except Exception:
        return FALLBACK_TFLOPS, FALLBACK_HBM_GBS, "fallback"


def host_threads() -> int:
    """Threads the CPU legs use: every core this process may run on (launchers such as torchrun
    set OMP_NUM_THREADS=1, which would otherwise serialise the CPU port)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def emitted_tokens(out_len: np.ndarray) -> int:
    return int(np.maximum(out_len[:, 0] - 2, 0).sum())


def cpu_leg(c, blobs, sents, n_sample: int, group: int, ensemble="prob_mean", repeat: int = 1):
    """Times the CPU restatement of the reference's math (the reference has no CPU forward path of its own
    and cannot be built without Boost and a GPU) on the first n_sample sentences of the batch, with all host
    threads.  group = 1 is the reference's own shape: one sentence at a time, rows = beam
    (src/decoder.h:1780-1840); group = 0 decodes the sample as one batch.  The dense products go through the
    Eigen headers the reference ships where that build is there, else through the restatement's own FMA loops."""
    from oracle import oracle_py
    gemm = "eigen" if oracle_py.eigen_lib() is not None else "canonical"
    sub = sents.subset(range(min(n_sample, sents.n)))
    best = None
    for _ in range(repeat):
        t0 = time.perf_counter()
        o = oracle_py.decode(c.desc, blobs, sub, beam=c.beam, nbest=1, lp_alpha=c.lp_alpha, cp_beta=c.cp_beta,
                             attention=c.attention, precision=c.precision, ensemble=ensemble, group=group,
                             threads=host_threads(), gemm=gemm)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    toks = emitted_tokens(o["len"])
    return {"value": toks / best, "seconds": best, "sentences": sub.n, "cores": host_threads(),
            "gemm": "Eigen 3.2.92 (the reference's vendored headers), OpenMP" if gemm == "eigen" else "the restatement's own blocked FMA loops, OpenMP"}


def cpu_baseline_block(c, blobs, sents, ensemble="prob_mean"):
    """cpu_baseline of the JSON line: the reference-shaped timing is the value; the batched one stands beside it."""
    ref = cpu_leg(c, blobs, sents, 4, 1, ensemble)
    bat = cpu_leg(c, blobs, sents, 16, 0, ensemble)
    return {"value": ref["value"], "unit": UNIT, "cores": ref["cores"], "kind": "port",
            "sample": f"first {ref['sentences']} sentences of the batch, one sentence at a time (rows = {c.beam}, the reference's own "
                      f"loop shape), {ref['seconds']:.1f} s of CPU work; dense products: {ref['gemm']}",
            "batched": {"value": bat["value"], "unit": UNIT,
                        "sample": f"first {bat['sentences']} sentences as one batch (rows = {bat['sentences']}*{c.beam}), {bat['seconds']:.1f} s of CPU work"}}


def run_reference(args):
    """The reference arm: the CPU restatement of the reference's math, in the reference's own loop shape (one
    sentence at a time), all host threads, a bounded sample of the same workload per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    c, batches = workload(args.workload, 0, 1)
    sents = batches[0]
    blobs = c.blobs()
    n_sample = 4
    times, toks, leg = [], 0, None
    for i in range(args.warmup + args.steps):
        leg = cpu_leg(c, blobs, sents, n_sample, 1)
        if i >= args.warmup:
            times.append(leg["seconds"])
            toks = leg["value"] * leg["seconds"]
        if sum(times) > 150:
            break
    steps_done = len(times)
    ms = 1e3 * sum(times) / steps_done
    value = toks / (ms / 1e3)
    sample = (f"first {n_sample} of the {sents.n} sentences of the batch per step, one sentence at a time (rows = {c.beam}), "
              f"all host threads; dense products: {leg['gemm']}")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps_done,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config_block(c, sents, args.gpus, args.workload),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": leg["cores"], "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference has no CPU forward path and cannot be built here (Boost, GPU-only math); this arm "
                "times the CPU restatement of its math (oracle/) in the reference's loop shape on the host cores",
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
        if os.environ.get("NCCL_DEBUG", "").upper() not in ("INFO", "TRACE"):
            os.environ["NCCL_DEBUG"] = "NONE"   # at VERSION / WARN the library prints its version banner to stdout, which carries the JSON line only
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    name = args.workload
    c, batches = workload(name, rank, world, args.precision, args.sentences)
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

    cls = {}   # kernel class -> [ms, launches] while kernel timing is on
    rec = {"flops": 0.0}

    def step_device():
        """One pass over this rank's batches, ids and outputs resident in HBM."""
        ms = 0.0
        for b, (d_ids, d_tok, d_len, d_score) in zip(batches, dbuf):
            dec.decode_device(d_ids.data_ptr(), b.off, b.steps, max_len, d_tok.data_ptr(), d_len.data_ptr(), d_score.data_ptr())
            st = dec.stats()
            ms += st["last_decode_ms"]
            rec["flops"] += st["last_rec_gemm_flops"]
            for k_, (m_, n_) in dec.kernel_times().items():
                e = cls.setdefault(k_, [0.0, 0])
                e[0] += m_; e[1] += n_
        return ms

    # ---- device-resident leg: `value` (no per-kernel events inside: they cost a few percent and end the
    # overlap of consecutive kernels at every event) ----
    for _ in range(args.warmup):
        step_device()
    s0 = dec.stats()
    barrier()
    clk_p, clk_path = clocks_start() if rank == 0 else (None, None)
    dev_ms = 0.0
    w0 = time.perf_counter()
    for _ in range(args.steps):
        dev_ms += step_device()
    barrier()
    wall_ms = 1e3 * (time.perf_counter() - w0)
    s1 = dec.stats()
    launches = s1["kernel_launches"] - s0["kernel_launches"]
    toks = sum(emitted_tokens(d[2].cpu().numpy()) for d in dbuf)
    row_steps = s1["decoder_row_steps"] - s0["decoder_row_steps"]
    sent_steps = s1["sentence_steps"] - s0["sentence_steps"]

    # ---- the same steps once more with a CUDA event before every kernel of the decoder steps: the roofline
    # figures of every kernel class (clock sampling runs on over this pass) ----
    dec.set_kernel_timing(True)
    cls.clear(); rec["flops"] = 0.0
    timed_ms = 0.0
    for _ in range(args.steps):
        timed_ms += step_device()
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
    dec.close()

    strong = None if args.no_strong_c3 else strong_c3(args, rank, world, local)

    # ---- reduce over ranks: max time, summed tokens ----
    vals = torch.tensor([dev_ms, wall_ms, e2e_wall_ms], dtype=torch.float64, device=dev)
    n_sent_local = sum(b.n for b in batches)
    positions_local = int(sum(int((b.steps + 1).sum()) for b in batches))
    sums = torch.tensor([toks, e_toks, launches, row_steps, n_sent_local], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    dev_ms, wall_ms, e2e_wall_ms = vals.tolist()
    toks_all, e_toks_all, launches_all, row_steps_all, n_sent_all = sums.tolist()

    if rank == 0:
        ms_per_step = dev_ms / args.steps
        value = toks_all * args.steps / (dev_ms / 1e3)
        e2e_value = e_toks_all * args.steps / (e2e_wall_ms / 1e3)
        H, V, L = c.desc.H, c.desc.V, c.desc.L
        Hp = (H + 63) // 64 * 64
        M = len(blobs)
        tf_peak, hbm_peak, peak_src = peaks()
        tensor = args.gemm_path != "simt"
        fp32 = c.precision != "bf16"
        nt = 2 if fp32 else 1                                     # 16-bit planes per operand on the tensor path
        gate_products = ({"tensor2": 4, "tensor3": 6}.get(args.gemm_path, 3) if fp32 else 1) if tensor else 0
        voc_products = ((4 if args.gemm_path in ("tensor2", "tensor3") else
                         (1 if args.gemm_path in ("tensor_v16", "tensor_v16x", "auto") and M == 1 else 3)) if fp32 else 1) if tensor else 0
        note = ("launch durations from a second pass over the same steps with a CUDA event before every kernel (the pass "
                "timed for `value` carries none); an event costs a few microseconds per launch and ends the overlap of "
                "consecutive kernels, so these durations are upper bounds. achieved = ALGORITHMIC flops or bytes; on the "
                "fp32 tensor path every product is computed as `products_per_product` 16-bit partial products, which is "
                "what tensor_pipe_* counts")
        total_cls_ms = sum(v[0] for v in cls.values()) or 1.0
        # one-product logits of a single fp32 model go out as fp16 (the library's default; LINMT_LOGITS16=0 keeps fp32)
        logits16 = tensor and fp32 and M == 1 and args.gemm_path in ("auto", "tensor_v16x") and os.environ.get("LINMT_LOGITS16", "1") != "0"

        def roof(key, kernel, bound, work, products=0):
            """Roofline block of one kernel class: algorithmic flops (tensor) or bytes (hbm) of the timed pass over
            the CUDA-event time of the class's launches."""
            ms, n = cls.get(key, [0.0, 0])
            if not n:
                return None
            peak = tf_peak if bound == "tensor" else hbm_peak
            ach = work / (ms / 1e3) / (1e12 if bound == "tensor" else 1e9)
            blk = {"bound": bound, "kernel": kernel, "achieved": ach, "peak": peak, "unit": "TFLOP/s" if bound == "tensor" else "GB/s",
                   "frac": ach / peak, "traffic": C2_TRAFFIC_BYTES.get(key) if name == "C2" and args.gemm_path == "auto" and fp32 else None,
                   "peak_source": peak_src, "launches": int(n), "avg_launch_ms": ms / n, "share_of_step": ms / total_cls_ms}
            if bound == "tensor":
                blk.update({"products_per_product": products, "tensor_pipe_tflops": ach * products if tensor else None,
                            "tensor_pipe_frac": ach * products / peak if tensor else None})
            return blk

        rs, ss = float(row_steps) , float(sent_steps)   # decoder forwards of a row / of a sentence in the timed pass
        blocks = [
            roof("lstm_gemm", f"decoder LSTM gate GEMMs [rows,2H]x[2H,4H] with the cell update in the epilogue ({args.gemm_path} path)",
                 "tensor", rec["flops"], gate_products),
            roof("vocab_gemm", f"vocabulary GEMM [rows,H]x[H,V] ({args.gemm_path} path)", "tensor", 2.0 * rs * H * V * M, voc_products),
            roof("attn_proj_gemm", "attention projections GEMM [rows,H]x[H,3H] (W_p | W_a^T | W_c2)", "tensor", 2.0 * rs * H * 3 * H * M, gate_products),
            roof("attn_out_gemm", "attention output GEMM [rows,H]x[H,H] (W_c1) + tanh", "tensor", 2.0 * rs * H * H * M, gate_products),
            roof("softmax_topk", "log-softmax statistics + per-row top-(k+1), one pass over the logits" + (" (fp16)" if logits16 else ""), "hbm",
                 rs * V * (2.0 if logits16 else 4.0)),
            roof("ensemble_combine", "ensemble combination of the members' distributions", "hbm", rs * V * 4.0 * (M + 1)),
            roof("gather", "beam reordering of the recurrent state (h planes of every layer, attentional state)", "hbm",
                 rs * (L + 1) * nt * Hp * 2.0 * 2 * M),
            roof("attention", "attention: p_t, window scores, softmax x Gaussian, weighted sum of W_c1-mapped states, tanh -> attentional state", "hbm",
                 (ss * 2 * 21 * Hp * 4.0 + rs * (3 * Hp * 4.0 + nt * Hp * 2.0)) * M),
            roof("beam_select", "beam selection (k(k+1) candidates per sentence)", "hbm", rs * (c.beam + 1) * 8.0),
        ]
        blocks = [b_ for b_ in blocks if b_]
        blocks.sort(key=lambda b_: -b_["share_of_step"])
        dominant, others = blocks[0], blocks[1:]
        dominant["note"] = note
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu = cpu_baseline_block(c, blobs, batches[0], ensemble)
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
            "roofline": dominant, "roofline_other": others,
            "cpu_baseline": cpu, "clocks": clocks, "gemm_path": args.gemm_path,
            "strong_c3": strong,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def strong_c3(args, rank, world, local):
    """The fixed job of the throughput configuration, strong-scaled: 4096 sentences of 10 to 80 words, bf16 weights,
    beam 12, length-bucketed batches of 128 dealt to the ranks by decoder forwards (shard.partition), every rank
    decoding its share on its own replica, and ONE gather of the hypotheses to rank 0 at the end -- all inside the
    timed region.  Rank 0 then decodes the whole job alone, so the speed-up is measured within this run."""
    import torch
    import torch.distributed as dist
    from linmt_b200 import decoder, shard
    c = synth.configs()["C3"]
    allsents = c.sentences(args.c3_sentences)
    batch = WORKLOADS["C3"][0]
    blobs = c.blobs()
    Tm = int(allsents.steps.max())
    dec = decoder.Decoder(c.desc, blobs, beam=c.beam, nbest=1, lp_alpha=c.lp_alpha, cp_beta=c.cp_beta, attention=c.attention,
                          precision="bf16", max_batch=batch, max_src_len=int(allsents.lengths().max()), max_steps=Tm, device=local)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def run(mine):
        """Decodes the sentences `mine` (indices into the job) batch by batch; returns the hypotheses as arrays
        (sentence index, padded token rows, lengths, scores) and the device time."""
        mine = np.asarray(mine, np.int64)
        sub = allsents.subset(mine)
        idx, toks, lens, scores, dev_ms = [], [], [], [], 0.0
        for b in shard.batches_by_length(sub, batch):
            o = dec.decode(sub.subset(b))
            dev_ms += dec.stats()["last_decode_ms"]
            t = np.zeros((len(b), Tm + 2), np.int32)
            t[:, :o["tok"].shape[2]] = o["tok"][:, 0]
            idx.append(mine[b]); toks.append(t); lens.append(o["len"][:, 0]); scores.append(o["score"][:, 0])
        return (np.concatenate(idx), np.concatenate(toks), np.concatenate(lens), np.concatenate(scores)), dev_ms

    def assemble(parts_list):
        tok = np.zeros((allsents.n, Tm + 2), np.int32); ln = np.zeros(allsents.n, np.int32); sc = np.zeros(allsents.n, np.float32)
        seen = 0
        for idx, t, l, s_ in parts_list:
            tok[idx] = t; ln[idx] = l; sc[idx] = s_; seen += len(idx)
        assert seen == allsents.n
        return tok, ln, sc

    parts = shard.partition(allsents, world, batch)
    warm, _ = run(parts[rank][:batch])   # warm-up: one batch, and one gather of its result
    shard.gather_parts(warm, dst=0)
    barrier()
    t0 = time.perf_counter()
    local_res, local_ms = run(parts[rank])
    t1 = time.perf_counter()
    gathered = shard.gather_parts(local_res, dst=0)
    merged = assemble(gathered) if rank == 0 else None
    barrier()
    wall = time.perf_counter() - t0
    fwd = float(sum(int(allsents.steps[i]) + 1 for i in parts[rank]))
    per = torch.tensor([[fwd, local_ms, float(len(parts[rank])), t1 - t0]], dtype=torch.float64, device=torch.device("cuda", local))
    if world > 1:
        allper = [torch.zeros_like(per) for _ in range(world)]
        dist.all_gather(allper, per)
        per = torch.cat(allper)
        wmax = torch.tensor([wall], dtype=torch.float64, device=per.device)
        dist.all_reduce(wmax, op=dist.ReduceOp.MAX)
        wall = float(wmax.item())
    out = None
    if rank == 0:
        toks = int(np.maximum(merged[1] - 2, 0).sum())
        out = {"workload": WORKLOADS["C3"][2], "sentences": allsents.n, "tokens": toks, "n_gpus": world,
               "seconds": wall, "value": toks / wall, "unit": UNIT, "scaling": "strong",
               "timed_region": "host ids in, every rank's batches through the host API, one gather of all hypotheses to rank 0",
               "per_rank": [{"rank": r, "sentences": int(per[r, 2].item()), "decoder_forwards": int(per[r, 0].item()),
                             "device_ms": float(per[r, 1].item()), "decode_wall_ms": 1e3 * float(per[r, 3].item())}
                            for r in range(per.shape[0])]}
    if world > 1:
        # the same job on one GPU, within this run: rank 0 alone
        barrier()
        if rank == 0:
            t0 = time.perf_counter()
            alone, _ = run(list(range(allsents.n)))
            alone = assemble([alone])
            torch.cuda.synchronize()
            w1 = time.perf_counter() - t0
            out["one_gpu_seconds"] = w1
            out["speedup_over_one_gpu"] = w1 / wall
            out["sentences_identical_to_one_gpu"] = int(((alone[0] == merged[0]).all(axis=1) & (alone[1] == merged[1])).sum())
        barrier()
    dec.close()
    return out


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
    ap.add_argument("--no-strong-c3", action="store_true", help="skip the strong-scaled C3 job reported beside the headline")
    ap.add_argument("--c3-sentences", type=int, default=4096)
    ap.add_argument("--sentences", type=int, default=None, help="cut a fixed job (C3-C5) down to its first N sentences (profiling captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
