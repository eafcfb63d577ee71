"""Benchmark of the PBS-Attn prefill attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--seq-len S] [--threshold T]

One step = one permuted_block_sparse_attn_fwd call (all stages) on the Llama-3.1-8B head shape at
131072 tokens (32 query / 8 KV heads, head_dim 128, bf16, block 128, segment 256, threshold 0.9,
seeded synthetic Q/K/V with planted heavy-hitter keys, sinks and RoPE).  With N > 1 the KV-head
groups are sharded over the ranks (strong scaling: the total work is fixed, and every N works on the
same seeded problem) and the step delivers the full (B, Hq, S, D) result to every rank: by default the
attention kernel stores each output tile into every rank's buffer over NVLink (--gather fused), else an
NCCL all-gather follows the call (--gather nccl).  Rank 0 prints one JSON line.

  value      selected-block TFLOP/s (4 * bs^2 * D per selected block) of the whole job, inputs
             resident in HBM, device time by CUDA events, max over ranks
  e2e        the same metric through the public API with HOST (pinned) q/k/v copied to the device
             and the output copied back inside the timed region
  roofline   the attention kernel alone: selected-block FLOPs / its event-timed duration, against the
             measured bf16 tensor peak (MEASURED_PEAKS.json)
  cpu_baseline  the CPU oracle (a port of the reference's PyTorch path) on a bounded sample

--impl reference times that CPU port on the host cores for the same metric and config.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from pbs_attn_b200.synth import WORKLOADS, Workload, make_qkv, make_qkv_heads  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum of one attn_tc_kernel launch on one GPU (bytes), from the ncu
# capture summarised in the named file under profiles/, with the commit whose kernel was captured: a later
# change of the kernel makes the figure stale until the capture is repeated.  Other workloads have none.
ATTN_KERNEL_DRAM_TRAFFIC = {
    "llama8b_heads_s131072": {"bytes": 20.20e9, "commit": "8ed0ae1", "profile": "profiles/attn_tc_kernel_llama8b_s32768.txt"},
}

METRIC = "prefill_attn_selected_block_tflops"
UNIT = "TFLOP/s"
CPU_SAMPLE = dict(q_heads=4, kv_heads=1, seq_len=32768)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_burst": p["bf16_tflops"],
                "bf16_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


def selected_flops(n_selected_blocks: float, w: Workload) -> float:
    return 4.0 * w.block_size * w.block_size * w.head_dim * n_selected_blocks


def dense_equiv_flops(w: Workload, q_heads: int) -> float:
    return 2.0 * w.batch * q_heads * float(w.seq_len) ** 2 * w.head_dim


class ClockSampler:
    """nvidia-smi in the background (read-only queries).  It is started well before the timed region,
    because it needs most of a second to deliver its first sample, and ``stop`` keeps the samples whose
    time stamps fall inside the region: the clock UNDER LOAD (this GPU runs into its power cap, so the
    loaded clock is the lower one)."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self, t0: float, t1: float):
        """Summary of the samples taken between the host times ``t0`` and ``t1`` (time.time())."""
        import datetime
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, power, smax, reasons, total = [], [], 0.0, set(), 0
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(c[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                clk, cmax = float(c[1]), float(c[2])
            except ValueError:
                continue
            total += 1
            smax = max(smax, cmax)
            if not (t0 <= ts <= t1):
                continue
            sm.append(clk)
            try:
                power.append(float(c[3]))
            except ValueError:
                pass
            for n, v in zip(names, c[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.file.close()
        os.unlink(self.file.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": smax or None, "reasons": [], "samples": 0, "samples_total": total}
        return {"sm_mhz": statistics.median(sm), "sm_min_mhz": min(sm), "sm_max_mhz": smax,
                "power_w": statistics.median(power) if power else None, "reasons": sorted(reasons),
                "samples": len(sm), "samples_total": total}


def cpu_port_run(w: Workload, seed: int):
    """One run of the CPU oracle on ``w``; returns (seconds, selected-block FLOPs)."""
    from oracle import pbs_oracle
    q, k, v = make_qkv(w, seed)
    t = time.perf_counter()
    r = pbs_oracle.permuted_block_sparse_attn_fwd(q, k, v, w.block_size, w.segment_size, w.threshold, stable=False)
    dt = time.perf_counter() - t
    n_sel = float(r.block_mask.sum()) if r.block_mask is not None else 0.0
    return dt, selected_flops(n_sel, w)


def sample_workload(w: Workload) -> Workload:
    s = dict(CPU_SAMPLE)
    s["seq_len"] = min(s["seq_len"], w.seq_len)
    s["kv_heads"] = 1
    s["q_heads"] = w.q_heads // w.kv_heads
    return w.with_(**s)


def sample_text(ws: Workload) -> str:
    return (f"{ws.q_heads} query heads / {ws.kv_heads} KV head of the workload at seq_len {ws.seq_len} "
            f"(one full call of the CPU port per step)")


def config_dict(w: Workload, world: int, extra=None):
    c = {"workload": w.name, "batch": w.batch, "q_heads": w.q_heads, "kv_heads": w.kv_heads,
         "head_dim": w.head_dim, "seq_len": w.seq_len, "block_size": w.block_size,
         "segment_size": w.segment_size, "threshold": w.threshold, "rope_theta": w.rope_theta,
         "hot_key_density": w.density, "sinks": w.sinks,
         "parallelism": f"kv-head groups sharded over {world} GPU(s), outputs all-gathered" if world > 1 else "single GPU",
         "l2": "inputs_exceed_l2"}
    if extra:
        c.update(extra)
    return c


# ------------------------------------------------------------------------------------ reference arm
def run_reference(args, w: Workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    ws = sample_workload(w)
    for i in range(args.warmup):
        if i == 0:
            cpu_port_run(ws, args.seed)          # one warm-up call is enough for a CPU path
    times, fl = [], 0.0
    for _ in range(args.steps):
        dt, fl = cpu_port_run(ws, args.seed)
        times.append(dt)
    total = sum(times)
    val = fl * len(times) / total / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
        "config": config_dict(w, 1, {"measured_on": "bounded sample, see sample_config"}),
        "same_config": False,
        "sample_config": {"q_heads": ws.q_heads, "kv_heads": ws.kv_heads, "seq_len": ws.seq_len, "batch": ws.batch,
                          "note": "the CPU port of the reference path (oracle/) is timed on one KV group at this length; "
                                  "value is a RATE (selected-block TFLOP/s), not the time of the full configuration"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample_text(ws)},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------ our arm
def run_ours(args, w: Workload):
    import torch.distributed as dist
    from pbs_attn_b200 import _cabi
    from pbs_attn_b200.prefill import get_plan, permuted_block_sparse_attn_fwd, permuted_block_sparse_attn_fwd_host
    from pbs_attn_b200.sharding import gather_heads, shard_heads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _cabi.load()
    peaks = load_peaks()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    # Every partition of the heads works on the same global problem: inputs are drawn per KV-head group.
    sh = shard_heads(w.q_heads, w.kv_heads, rank, world)
    q, k, v = make_qkv_heads(w, args.seed, sh.kv_start, sh.kv_count, sh.q_start, sh.q_count, device=dev)
    torch.cuda.synchronize()

    # ---- how the full (B, Hq, S, D) result reaches every rank
    gather_mode, gather_note, fused = "none", None, None
    if world > 1:
        gather_mode = args.gather
        if gather_mode == "fused":
            try:
                from pbs_attn_b200.peer_gather import FusedHeadGather, permuted_block_sparse_attn_fwd_gathered
                fused = FusedHeadGather(w.batch, w.q_heads, w.kv_heads, w.seq_len, w.head_dim, q.dtype, dev)
            except Exception as e:      # e.g. CUDA IPC not permitted on this host: the NCCL all-gather still works
                gather_mode, gather_note = "nccl", f"fused gather unavailable: {e}"

    def step():
        if fused is not None:
            return permuted_block_sparse_attn_fwd_gathered(fused, q, k, v, w.block_size, w.segment_size, w.threshold)
        out = permuted_block_sparse_attn_fwd(q, k, v, w.block_size, w.segment_size, w.threshold, True)
        if world > 1:
            out = gather_heads(out, w.q_heads, w.kv_heads)
        return out

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        out = step()
    barrier()
    plan = get_plan(q, sh.kv_count, w.block_size, w.segment_size)
    plan.check_status()
    n_sel_local = float(plan.block_mask.sum().item())

    launches0 = lib.pbs_launch_count()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    barrier()
    t_timed0 = time.time()
    ev[0].record()
    for _ in range(args.steps):
        out = step()
    ev[1].record()
    barrier()
    t_timed1 = time.time()
    launches = lib.pbs_launch_count() - launches0
    ms_total = ev[0].elapsed_time(ev[1])
    plan.check_status()

    # ---- N > 1, outside the timed region: is the gathered tensor right?
    gather_check = None
    if world > 1:
        local = permuted_block_sparse_attn_fwd(q, k, v, w.block_size, w.segment_size, w.threshold, True)
        torch.cuda.synchronize()
        own_equal = bool(torch.equal(out[:, sh.q_slice], local))
        # a head this rank does not own, recomputed here from regenerated inputs: the next rank's first head
        other = shard_heads(w.q_heads, w.kv_heads, (rank + 1) % world, world)
        fq, fk, fv = make_qkv_heads(w, args.seed, other.kv_start, 1, other.q_start, 1, device=dev)
        foreign = permuted_block_sparse_attn_fwd(fq, fk, fv, w.block_size, w.segment_size, w.threshold, True)
        torch.cuda.synchronize()
        fd = (out[:, other.q_start:other.q_start + 1].float() - foreign.float()).abs().max().item()
        ok = torch.tensor([int(own_equal), int(fd <= 2e-2)], dtype=torch.int32, device=dev)
        fmax = torch.tensor([fd], dtype=torch.float64, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        dist.all_reduce(fmax, op=dist.ReduceOp.MAX)
        gather_check = {"own_slice_bit_equal_on_all_ranks": bool(ok[0].item()),
                        "foreign_head_recomputed_max_abs_over_ranks": float(fmax.item()),
                        "foreign_head_within_tolerance_on_all_ranks": bool(ok[1].item())}
        del local, foreign, fq, fk, fv
        plan = get_plan(q, sh.kv_count, w.block_size, w.segment_size)

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty(w.batch, sh.q_count, w.seq_len, w.head_dim, dtype=q.dtype).pin_memory()

    def e2e_step():
        permuted_block_sparse_attn_fwd_host(hq, hk, hv, w.block_size, w.segment_size, w.threshold, True, out=ho,
                                            device=dev)

    e2e_step()
    barrier()
    e2e_steps = max(1, args.steps)
    ev2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev2[0].record()
    for _ in range(e2e_steps):
        e2e_step()
    ev2[1].record()
    barrier()
    e2e_ms_total = ev2[0].elapsed_time(ev2[1])
    clocks = sampler.stop(t_timed0, t_timed1) if rank == 0 else None

    # ---- per-stage device times on this rank (the attention kernel gives the roofline)
    plan = get_plan(q, sh.kv_count, w.block_size, w.segment_size)
    opt = plan.options(w.threshold)
    o2 = torch.empty_like(q)
    stage_calls = [
        ("key_importance", lambda: plan.key_importance(q, k)),
        ("segment_permute", lambda: plan.segment_permute(k, v)),
        ("pool_queries", lambda: plan.pool_queries(q)),
        ("select_blocks", lambda: plan.select_blocks(opt)),
        ("tile_lists", lambda: plan.build_tile_lists()),
        ("attention", lambda: plan.attn_fwd(q, o2)),
    ]
    reps = max(1, min(args.steps, 3))
    stage_ms = {}
    for name, fn in stage_calls:
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        stage_ms[name] = a.elapsed_time(b) / reps
    plan.check_status()

    # ---- reduce over ranks: time = max, work = sum
    t = torch.tensor([ms_total, e2e_ms_total, stage_ms["attention"]], dtype=torch.float64, device=dev)
    work = torch.tensor([n_sel_local], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(work, op=dist.ReduceOp.SUM)
    ms_total, e2e_ms_total, attn_ms_max = (float(x) for x in t.tolist())
    n_sel = float(work.item())

    if rank == 0:
        ms_step = ms_total / args.steps
        fl_sel = selected_flops(n_sel, w)
        fl_dense = dense_equiv_flops(w, w.q_heads)
        nb = -(-w.seq_len // w.block_size)
        causal_blocks = w.batch * w.q_heads * nb * (nb + 1) / 2
        value = fl_sel / (ms_step * 1e-3) / 1e12
        e2e_ms = e2e_ms_total / e2e_steps
        e2e_val = fl_sel / (e2e_ms * 1e-3) / 1e12
        esz = q.element_size()
        h2d = w.batch * (w.q_heads + 2 * w.kv_heads * max(1, world // w.kv_heads)) * w.seq_len * w.head_dim * esz
        d2h = w.batch * w.q_heads * w.seq_len * w.head_dim * esz
        # attention kernel of THIS rank: its own selected blocks over its own duration
        attn_s = stage_ms["attention"] * 1e-3
        achieved = selected_flops(n_sel_local, w) / attn_s / 1e12
        B, Hq, Hkv, S, D, bs = w.batch, sh.q_count, sh.kv_count, w.seq_len, w.head_dim, w.block_size
        L = (S // w.segment_size) * w.segment_size
        stage_bytes = {      # algorithmic HBM bytes per launch group (this rank's heads)
            "key_importance": B * Hkv * L * D * esz + B * Hq * bs * D * esz + 4 * B * Hq * L,
            "segment_permute": 2 * B * Hkv * S * D * esz + 4 * B * Hq * L + 2 * B * Hq * S * D * esz + 4 * B * Hq * S + B * Hq * nb * D * esz,
            "pool_queries": B * Hq * S * D * esz + B * Hq * nb * D * esz,
            "select_blocks": 2 * B * Hq * nb * D * esz + B * Hq * nb * nb,
            "tile_lists": B * Hq * nb * nb + 4 * B * Hq * ((S + 255) // 256) * ((S + 127) // 128),
        }
        stages = {n: {"ms": round(ms, 4)} for n, ms in stage_ms.items()}
        for n, by in stage_bytes.items():
            stages[n]["gbs"] = round(by / (stage_ms[n] * 1e-3) / 1e9, 1)
            stages[n]["frac_hbm"] = round(stages[n]["gbs"] / peaks["hbm_gbs"], 4)
        traffic = ATTN_KERNEL_DRAM_TRAFFIC.get(w.name) if world == 1 else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
            "config": config_dict(w, world, {"gather": gather_mode}),
            "selected_tflop_per_step": fl_sel / 1e12, "dense_equiv_tflop_per_step": fl_dense / 1e12,
            "dense_equiv_tflops": fl_dense / (ms_step * 1e-3) / 1e12,
            "frac_bf16_burst_peak_whole_call_per_gpu": value / world / peaks["bf16_burst"],
            "e2e": {"value": e2e_val, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps},
            "gpu_launches": int(launches),
            # frac is ALWAYS against the sustained measured peak (the kernel is timed back to back, at N = 1 it
            # runs at the power cap); frac_burst is the same figure against the burst peak
            "roofline": {"kernel": "attn_tc_kernel", "bound": "tensor", "achieved": achieved,
                         "peak": peaks["bf16_sustained"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_sustained"],
                         "frac_sustained": achieved / peaks["bf16_sustained"], "frac_burst": achieved / peaks["bf16_burst"],
                         "peak_burst": peaks["bf16_burst"], "peak_source": f"{peaks['source']} (sustained)",
                         "traffic": traffic["bytes"] if traffic else None,
                         "traffic_source": (f"ncu, {traffic['profile']}, kernel as of commit {traffic['commit']}" if traffic else None),
                         "traffic_unit": "bytes per launch",
                         "kernel_ms": stage_ms["attention"], "kernel_ms_max_over_ranks": attn_ms_max,
                         "density": n_sel / causal_blocks, "stages": stages},
            "clocks": clocks,
        }
        if gather_check is not None:
            line["gather_check"] = gather_check
        if gather_note:
            line["gather_note"] = gather_note
        if world == 1 and not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count() or 1)
            ws = sample_workload(w)
            dt, fl = cpu_port_run(ws, args.seed)
            line["cpu_baseline"] = {"value": fl / dt / 1e12, "unit": UNIT, "cores": torch.get_num_threads(),
                                    "kind": "port", "seconds": dt, "sample": sample_text(ws)}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        if fused is not None:
            fused.close()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama8b_heads_s131072", choices=sorted(WORKLOADS))
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--threshold", type=float, default=None)
    ap.add_argument("--block-size", type=int, default=None, help="selection block size (64 or 128)")
    ap.add_argument("--segment-size", type=int, default=None, help="permutation segment size")
    ap.add_argument("--density", type=float, default=None, help="fraction of key positions planted as heavy hitters")
    ap.add_argument("--heads", default=None, metavar="HQ,HKV",
                    help="run a slice of the workload with this many query / KV heads (for profiler-sized cases)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: outputs stored into every rank's full tensor by the attention kernel over NVLink "
                         "(fused, the default), or an NCCL all-gather after the call")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.seq_len:
        w = w.with_(seq_len=args.seq_len, name=f"{w.name.rsplit('_s', 1)[0]}_s{args.seq_len}")
    if args.threshold is not None:
        w = w.with_(threshold=args.threshold)
    if args.block_size:
        w = w.with_(block_size=args.block_size, name=f"{w.name}_bs{args.block_size}")
    if args.segment_size:
        w = w.with_(segment_size=args.segment_size, name=f"{w.name}_seg{args.segment_size}")
    if args.density is not None:
        w = w.with_(density=args.density)
    if args.heads:
        hq, hkv = (int(x) for x in args.heads.split(","))
        w = w.with_(q_heads=hq, kv_heads=hkv, name=f"{w.name}_h{hq}x{hkv}")
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
