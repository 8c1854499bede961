#!/usr/bin/env python3
"""Benchmark of the quantized decode path: Q4_K x Q8_K GEMVs of a Mistral-7B-shaped layer set,
32 layers, batch 1 (seeded synthetic weights and activations).

    python bench.py --gpus 1 --steps K --warmup W            # this library (CUDA kernels)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU code

A step is one pass over the 7 x 32 GEMVs.  The metric is effective HBM bandwidth: algorithmic
bytes (quantized weights + fp32 activations in + fp32 outputs out) divided by device time.
The default schedule runs the step as persistent launches of 112 products each, replayed from a
CUDA graph.  With N GPUs every rank holds a layer set of the same size (its row shard of an
N-times larger model), runs the same step, and the ranks' output slices are exchanged by stores
from the product kernel into every rank's gathered buffer (or, --exchange nccl, by an all-gather);
the value is the sum of the ranks' bytes over the slowest rank's time (weak scaling).

One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from bpd_substrate_b200 import synth  # noqa: E402

METRIC = "Q4_K x Q8_K GEMV effective HBM bandwidth"
UNIT = "GB/s"
WORKLOAD = "mistral7b_layer_set_x32_q4k_decode_batch1"
N_LAYERS = 32
KERNEL_OF = {"persistent": "k_gemv_stream_q4k_q8k", "batched": "k_gemv_batch_q4k_q8k", "grouped": "k_gemv_q4k_q8k", "separate": "k_gemv_q4k_q8k",
             "chain": "k_gemv_batch_q4k_q8k", "chain4": "k_gemv_batch_q4k_q8k", "chain-separate": "k_gemv_batch_q4k_q8k",
             "chain-persistent": "k_decode_chain"}
# DRAM traffic / algorithmic bytes of each schedule's dominant kernel, from profiler captures of a 4-layer
# case (dram__bytes_read.sum + dram__bytes_write.sum per launch): nothing is re-read
TRAFFIC_PER_ALGORITHMIC = {"persistent": 1.008, "batched": 1.03, "grouped": 1.00, "separate": 1.00, "chain": 1.03, "chain4": 1.03,
                           "chain-separate": 1.03, "chain-persistent": 1.03}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 8:
                continue
            try:
                sm.append(float(r[0]))
                smax.append(float(r[1]))
            except ValueError:
                continue
            for name, val in zip(names, r[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(np.max(smax)) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_activations(ls, seed):
    rng = np.random.default_rng(seed)
    return rng.standard_normal(ls.x_bytes // 4, dtype=np.float32)


# --------------------------------------------------------------------------- CPU baseline

def cpu_reference_run(steps, warmup, layers_per_step, threads):
    """Times the reference's own bpd_qmatmul_q4k (bench/bpd_quant.c:88-109 of the reference,
    compiled unmodified) over `layers_per_step` layers of the workload, rows split over
    `threads` host threads.  Falls back to this repository's C restatement when the compiled
    reference is not present.  Returns (GB/s, kind, seconds per step)."""
    import ctypes as C
    from concurrent.futures import ThreadPoolExecutor
    from oracle import binding
    if binding.ref_available("bpd_quant.so"):
        lib = binding.load_ref("bpd_quant.so")
        kind = "reference"

        def gemv(w, x, out, rows, cols):
            lib.bpd_qmatmul_q4k(w, x, out, rows, cols)
    else:
        orc = binding.Oracle()
        kind = "port"

        def gemv(w, x, out, rows, cols):
            orc.lib.orc_qmatmul_q4k(w, x, out, rows, cols, 0)
    rng = np.random.default_rng(2000)
    base = []
    nbytes = 0
    for name, rows, cols in synth.MISTRAL_LAYER:
        base.append((synth.q4k_matrix(rows, cols, rng), synth.activations(cols, rng), np.zeros(rows, np.float32), rows, cols))
        nbytes += synth.gemv_bytes_q4k(rows, cols)
    nbytes *= layers_per_step
    # every layer of the step has its own weight bytes, as on the GPU (layer l = the base matrices rotated by
    # l + 1 super-blocks): 3.9 GB for 32 layers, streamed from host memory once per step
    layers = []
    for layer in range(layers_per_step):
        layers.append([(np.roll(w, synth.Q4K_BYTES * (layer + 1)) if layers_per_step > 1 else w, x, out, rows, cols)
                       for w, x, out, rows, cols in base])
    pool = ThreadPoolExecutor(threads)

    def one_layer(mats):
        jobs = []
        for w, x, out, rows, cols in mats:
            rb = synth.q4k_row_bytes(cols)
            per = (rows + threads - 1) // threads
            for t in range(threads):
                r0, r1 = t * per, min(rows, (t + 1) * per)
                if r0 < r1:
                    jobs.append(pool.submit(gemv, w.ctypes.data + r0 * rb, x.ctypes.data,
                                            out.ctypes.data + 4 * r0, r1 - r0, cols))
        for j in jobs:
            j.result()

    for _ in range(warmup):
        for mats in layers:
            one_layer(mats)
    t0 = time.perf_counter()
    for _ in range(steps):
        for mats in layers:
            one_layer(mats)
    dt = (time.perf_counter() - t0) / steps
    pool.shutdown()
    return nbytes / dt / 1e9, kind, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    # a step is the whole workload (32 layers, 224 GEMVs), about 0.6 s on 16 threads; the number of timed steps is
    # bounded so that the run ends within a few minutes whatever --steps says
    steps, warmup = max(1, min(args.steps, 100)), max(1, min(args.warmup, 3))
    value, kind, dt = cpu_reference_run(steps, warmup, N_LAYERS, threads)
    sample = (f"the whole step (32 layers, 224 GEMVs, 6,979,321,856 weights) {steps} times, W4A32 bpd_qmatmul_q4k of the "
              f"reference (the only Q4_K GEMV it has), rows split over {threads} host threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": N_LAYERS, "gemvs_per_step": 7 * N_LAYERS, "tokens": 1, "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm

def check_layer(ls, x_all, layer, schedule):
    """Runs the step once more and compares every product of one layer with the CPU checker (Q8_K
    quantization and the Q4_K x Q8_K dot in binary64): norm-wise max|d| / max|ref| per product."""
    from oracle.binding import Oracle
    orc = Oracle()
    ls.upload_activations(x_all)
    ls.step(schedule)
    out_all = ls.download_outputs()
    worst = 0.0
    for m, (_, rows, cols) in enumerate(ls.local):
        T = ls.tokens
        x = ls.activation_slice(x_all, layer, m).reshape(T, cols)
        got = ls.output_slice(out_all, layer, m).reshape(T, rows)
        _, ref64 = orc.qmm_q4k_q8k(ls.host_weight(layer, m), x, T, rows, cols)
        worst = max(worst, float(np.max(np.abs(got - ref64)) / np.max(np.abs(ref64))))
    return {"layer": layer, "products": len(ls.local), "max_norm_err": worst, "tolerance": 1e-5, "ok": bool(worst <= 1e-5),
            "against": "CPU checker: Q8_K quantizer + Q4_K x Q8_K dot, binary64 sum"}


def run_gpu(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    from bpd_substrate_b200 import capi
    from bpd_substrate_b200.dispatch import LayerSet
    lib = capi.load()
    dist = torch = None
    if world > 1:
        # keep stdout to the one JSON line (NCCL announces its version there at the default level)
        os.environ.setdefault("NCCL_DEBUG", "WARN")
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    capi.check(lib.bpdq_set_device(local_rank), "set device")
    lib.bpdq_clear_status()

    # Every rank holds a full-size layer set: its row shard of a `world`-times larger model.
    out_local = None
    if args.workload == "llama70b":
        # one model for all ranks: rank r owns rows [r*N/world, (r+1)*N/world) of every matrix; the
        # output head rides along as an eighth matrix of every 80th layer's worth of work
        shapes, shard = synth.LLAMA70B_LAYER, (rank, world)
    else:
        shapes, shard = synth.MISTRAL_LAYER, (0, 1)
    if world > 1:
        # NCCL reads this rank's output arena directly: let torch own that allocation
        o_floats = args.tokens * args.layers * sum(rows // shard[1] for _, rows, _ in shapes)
        out_local = torch.empty(o_floats, dtype=torch.float32, device="cuda")
    schedule = args.schedule
    chain = schedule in ("chain", "chain4", "chain-separate", "chain-persistent")
    if chain:
        # the same seven matrices per layer as a DEPENDENT chain (every product reads what the step
        # before it wrote), with the elementwise steps of the reference's decode loop in between
        if world > 1 or args.workload != "mistral7b" or args.tokens != 1:
            raise SystemExit("--schedule chain: one GPU, mistral7b shapes, one token")
        from bpd_substrate_b200.dispatch import DecodeChain
        ls = DecodeChain(n_layers=args.layers, seed=2000)
    else:
        ls = LayerSet(shapes, args.layers, seed=2000 + (rank if args.workload == "mistral7b" else 0), row_shard=shard,
                      d_out=out_local.data_ptr() if out_local is not None else None, tokens=args.tokens)
    ls.even_ranges = bool(args.even_ranges)
    step_bytes = ls.algorithmic_bytes()
    launches = ls.launches_per_step(schedule)
    # launches of the dominant kernel (the batched schedule adds one small quantizer per layer,
    # which overlaps the previous GEMV kernel and is counted in the step time)
    main_launches = launches // 2 if schedule == "persistent" else args.layers if schedule == "batched" else (
        1 if schedule == "chain-persistent" else
        (7 if schedule == "chain-separate" else 4) * args.layers if chain else launches)
    x_host = lib.bpdq_host_alloc(ls.x_bytes)
    o_host = lib.bpdq_host_alloc(ls.o_bytes)
    x_np = np.ctypeslib.as_array((np.ctypeslib.ctypes.c_float * (ls.x_bytes // 4)).from_address(x_host))
    x_np[:] = make_activations(ls, 3000 + rank)
    ls.upload_activations(x_np)
    ls.capture(schedule)

    gathered = ext_stream = comm_stream = None
    chunks = [(0, args.layers)]
    if world > 1:
        # All-gather of the ranks' output slices (the exchange step of row sharding).  The step is cut
        # into chunks of layers; the gather of a chunk runs on a second stream under the GEMVs of the
        # next chunk, and the compute stream joins it before the step ends, so that one pair of CUDA
        # events on the compute stream spans GEMVs and exchange.
        n_chunks = max(1, min(args.gather_chunks, args.layers)) if not chain else 1
        bounds = [args.layers * c // n_chunks for c in range(n_chunks + 1)]
        chunks = [(bounds[c], bounds[c + 1]) for c in range(n_chunks)]
        gathered = torch.empty(world * (ls.o_bytes // 4), dtype=torch.float32, device="cuda")
        ext_stream = torch.cuda.ExternalStream(ls.stream)
        comm_stream = torch.cuda.Stream()
        for c in chunks:
            ls.capture(schedule, c if len(chunks) > 1 else None)

    # The exchange without a collective: the product kernels store their results into every rank's gathered
    # buffer themselves (peer memory), and a flag per rank and step replaces the all-gather's rendezvous.
    peer = None
    if world > 1 and args.exchange == "peer" and schedule in ("batched", "persistent") and args.tokens == 1:
        from bpd_substrate_b200.peer import PeerExchange
        try:
            peer = PeerExchange(lib, dist, rank, world, ls.o_bytes)
            for parity in (0, 1):
                peer.register(ls.d_out, parity)
                ls.capture(schedule, tag=parity)
                for r in ls.host_ranges(args.copy_chunks):      # the end-to-end leg replays ranges of layers
                    ls.capture(schedule, r, tag=parity)
            peer.unregister()
        except Exception as exc:            # set-up fails on all ranks or on none (PeerExchange agrees on it)
            sys.stderr.write(f"rank {rank}: {exc}; using the NCCL all-gather\n")
            lib.bpdq_clear_status()
            peer = None
        if peer is not None:
            chunks = [(0, args.layers)]
    steps_done = [0]

    ev0, ev1 = lib.bpdq_event_create(), lib.bpdq_event_create()

    def barrier():
        if world > 1:
            dist.barrier()
        lib.bpdq_sync()

    def exchange_all():
        if world > 1:
            with torch.cuda.stream(ext_stream):
                dist.all_gather_into_tensor(gathered, out_local)

    def step_with_exchange():
        """One step's GEMVs and the all-gather of their outputs."""
        if world == 1:
            ls.step(schedule)
            return
        if peer is not None:
            ls.step(schedule, tag=steps_done[0] & 1)
            peer.signal_and_wait(ls.stream)      # this rank's gathered buffer of the step's parity is complete
            steps_done[0] += 1
            return
        g_off = 0
        for c in chunks:
            ls.step(schedule, c if len(chunks) > 1 else None)
            begin, nbytes = ls.layer_output_range(*c)
            done = torch.cuda.Event()
            done.record(ext_stream)
            comm_stream.wait_event(done)
            with torch.cuda.stream(comm_stream):
                dist.all_gather_into_tensor(gathered[g_off:g_off + world * (nbytes // 4)],
                                            out_local[begin // 4:(begin + nbytes) // 4])
            g_off += world * (nbytes // 4)
        ext_stream.wait_stream(comm_stream)

    # ---- device-resident timing: inputs already in HBM
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    for _ in range(args.warmup):
        step_with_exchange()
    barrier()
    lib.bpdq_event_record(ev0, ls.stream)
    for _ in range(args.steps):
        step_with_exchange()
    lib.bpdq_event_record(ev1, ls.stream)
    ms_total = lib.bpdq_event_elapsed_ms(ev0, ev1)
    barrier()
    # GEMV-only device time (no exchange), for the roofline of the kernel itself
    lib.bpdq_event_record(ev0, ls.stream)
    for _ in range(args.steps):
        ls.step(schedule)
    lib.bpdq_event_record(ev1, ls.stream)
    ms_kernel_total = lib.bpdq_event_elapsed_ms(ev0, ev1)
    # The timed region can be shorter than one period of the clock sampler: keep the same steps running for
    # half a second more (untimed) so that the record holds samples taken under this very load.
    clocks = None
    if rank == 0:
        t_soak = time.perf_counter()
        while time.perf_counter() - t_soak < 0.5:
            for _ in range(20):
                ls.step(schedule)
            lib.bpdq_stream_sync(ls.stream)
        clocks = sampler.stop()
        clocks["window"] = "warm-up, the timed steps and 0.5 s of the same steps after them, sampled every 20 ms"

    # ---- one layer of the step against the CPU checker (rank 0; the checker is never the thing measured)
    check = None
    if rank == 0 and not chain and not args.no_check:
        check = check_layer(ls, x_np, args.layers // 2, schedule)

    # ---- end to end through the public call with HOST buffers
    def host_step():
        """Copies in, products, exchange of the output slices, copies out; returns when everything has finished."""
        if chain:
            ls.step_host(x_host, o_host, schedule)
        elif peer is not None:
            def flags():
                peer.signal_and_wait(ls.stream)
            ls.step_host(x_host, o_host, schedule, chunks=args.copy_chunks, tag=steps_done[0] & 1, after=flags)
            steps_done[0] += 1
        else:
            ls.step_host(x_host, o_host, schedule, chunks=args.copy_chunks)
            exchange_all()
            if world > 1:
                ext_stream.synchronize()

    for _ in range(min(args.warmup, 3)):
        host_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        host_step()
    t_e2e = time.perf_counter() - t0

    ms_step = ms_total / args.steps
    ms_kernel = ms_kernel_total / args.steps
    if world > 1:
        t = torch.tensor([ms_step, ms_kernel, t_e2e], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, ms_kernel, t_e2e = (float(v) for v in t.tolist())
    status = lib.bpdq_last_status()

    if rank == 0:
        peak, peak_kind = measured_peak()
        total_bytes = step_bytes * world
        if args.tokens > 1:
            # several activation rows per product: the batched multi-token kernel where the schedule is batched
            kernel_name = ls.multi_token_kernel(schedule)
            traffic = None
        else:
            kernel_name = KERNEL_OF[schedule]
            traffic = TRAFFIC_PER_ALGORITHMIC[schedule] * step_bytes / main_launches
        value = total_bytes / (ms_step * 1e-3) / 1e9
        achieved = step_bytes / (ms_kernel * 1e-3) / 1e9      # per GPU, kernel only
        e2e_value = total_bytes / (t_e2e / args.steps) / 1e9
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            v, kind, dt = cpu_reference_run(1, 1, 32, threads)
            cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": kind,
                   "sample": "one full step (32 layers, 224 GEMVs), W4A32 bpd_qmatmul_q4k of the reference, rows "
                             f"split over {threads} host threads, {dt:.2f} s wall"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak" if args.workload == "mistral7b" else "strong",
            "vs_baseline": None, "dtype": "int8 dot, f32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD if args.workload == "mistral7b" else
                       f"llama70b_layer_set_x{args.layers}_q4k_decode_batch{args.tokens}_rowshard{world}",
                       "layers": args.layers, "gemvs_per_step": 7 * args.layers, "tokens": args.tokens,
                       "schedule": schedule, "launches_per_step": launches + (1 if peer is not None else 0),
                       "weights_bytes_per_gpu": ls.weight_bytes,
                       "dependencies": "chain: every product reads the previous step's output" if chain else
                       "independent products, inputs resident before the step",
                       "l2": "inputs larger than L2: 3.9 GB of weights stream through once per step",
                       "parallelism": f"row-shard x{world}" if world > 1 else "single GPU",
                       "exchange": ("none: the product kernels store every result into all ranks' gathered buffers over NVLink "
                                    "(peer memory, double-buffered by step parity); one flag per rank and step, bounded wait"
                                    if peer is not None else
                                    f"NCCL all-gather of output slices in {len(chunks)} chunks of layers per step, each under "
                                    "the next chunk's GEMVs" if len(chunks) > 1 else
                                    "NCCL all-gather of output slices once per step") if world > 1 else "none"},
            "pct_of_peak": 100.0 * value / (peak * world),
            "elements_per_s": (ls.weight_bytes / synth.Q4K_BYTES * 256) * world / (ms_step * 1e-3),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)",
                         "kernel": kernel_name, "traffic": traffic,
                         "traffic_source": "ncu dram__bytes_read+write per launch / algorithmic bytes, 4-layer capture "
                                           "(profiles/), scaled by bytes",
                         "algorithmic_bytes_per_launch": step_bytes / main_launches,
                         "avg_launch_us": ms_kernel * 1e3 / main_launches},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": ls.x_bytes * world,
                    "d2h_bytes_per_step": ls.o_bytes * world},
            "gpu_launches": (launches + (1 if peer is not None else 0)) * args.steps,   # + the flag kernel of a step
            "clocks": clocks,
            "status": status,
        }
        if check:
            line["check"] = check
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    ls.close()                     # (destroys the graphs that store to the peers' buffers)
    if world > 1:
        if peer is not None:
            peer.close(dist)
        dist.barrier()
        dist.destroy_process_group()
    if status != 0:
        sys.exit(1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--schedule", default="persistent", choices=["persistent", "batched", "grouped", "separate", "chain", "chain4", "chain-separate",
                                                                  "chain-persistent"],
                    help="persistent: the benchmark (the step's independent products as persistent launches of 112 products "
                         "whose weight stream never drains); batched: a layer's seven products per launch; grouped / "
                         "separate: fewer products per launch; chain: the seven products as a dependent decode chain, "
                         "rms_norm / SwiGLU as small kernels writing quantized records, residual add in the product's "
                         "epilogue (8 launches per layer); chain4: the steps inside the product kernels (4); "
                         "chain-separate: the reference's 13-call sequence per layer; chain-persistent: the whole token as "
                         "one cooperative launch with grid-wide barriers between dependent phases")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison of one layer with the CPU checker")
    ap.add_argument("--even-ranges", action="store_true", help="end-to-end leg: ranges of equal size instead of tapered ones")
    ap.add_argument("--copy-chunks", type=int, default=4,
                    help="end-to-end leg: ranges of layers whose host copies run on their own streams under the other "
                         "ranges' GEMVs (1: copy in, step, copy out in sequence)")
    ap.add_argument("--exchange", choices=("peer", "nccl"), default="peer",
                    help="N > 1 GPUs: peer = the product kernels store their results into every rank's gathered buffer "
                         "(no collective; schedule batched); nccl = one all-gather per step")
    ap.add_argument("--gather-chunks", type=int, default=1,
                    help="N > 1 GPUs: 1 = one all-gather after the step's GEMVs (default); more = the gather is cut into "
                         "chunks of layers, each on a second stream under the next chunk's GEMVs (measured slower at 2 GPUs: "
                         "0.783 ms against 0.753 ms per step, the NCCL kernels compete with CTAs that fill every SM)")
    ap.add_argument("--workload", default="mistral7b", choices=["mistral7b", "llama70b"],
                    help="mistral7b: the benchmark (every rank a full layer set, weak scaling); llama70b: the "
                         "70B-shaped model row-sharded over the ranks (80 layers + output head, strong scaling)")
    ap.add_argument("--tokens", type=int, default=1, help="activation rows per product (llama70b sweep: 1 and 8)")
    ap.add_argument("--layers", type=int, default=None,
                    help="layers resident (32 is the benchmark; fewer only for profiler captures)")
    args = ap.parse_args()
    if args.layers is None:
        args.layers = N_LAYERS if args.workload == "mistral7b" else 80
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
