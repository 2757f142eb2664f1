#!/usr/bin/env python
"""Throughput of one full training step (forward, output error, backward, derivative-weight accumulation, optimizer
update) on the wide-MLP workload: 8 x FC 4096 + BatchNorm + ReLU + inverted dropout 0.5, FC 4096 -> 1024, MSE, Adam,
GLOBAL batch 4096, fp32 (split-precision tensor-core contractions), synthetic seeded data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1|c3|c4|c5]
    python bench.py --gemm M N K [--steps K]          one contraction through the C ABI (error against float64 + timing)

N > 1 is launched by torchrun, one rank per GPU.  The global batch of the configuration is SHARDED over the ranks
(strong scaling, as the configuration states it): every rank runs the step on 1/N of the rows, derivatives are summed
with NCCL and batch-norm statistics are synchronised, so the result equals the one-GPU step.  The line also carries,
under extra keys, the same step with the configuration's batch PER GPU (weak scaling), a correctness check of the
data-parallel path (`dp_check`), and at N = 1 the other recurrent workload (`other_workloads`).
Prints ONE JSON line.  `value` is measured with inputs resident in HBM; `e2e` goes through the host-buffer entry
points (host -> device copy of inputs and targets and a device -> host read of the loss inside the timed region).
`--impl reference` times the reference's own CPU/OpenMP implementation (compiled into oracle/_ref) on the host cores,
on a bounded sample of the same workload.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

CLASS_NAMES = ["gemm", "split", "normalization", "elementwise", "optimizer", "recurrent", "comm", "other"]
CPU_SAMPLE_ROWS = {"c2": 64, "c1": 128, "c3": 16, "c4": 64, "c5": 4}


def _peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """samples SM clocks and throttle reasons with nvidia-smi while the timed region runs"""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.proc, self.lines = device, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_run(wl_name, steps, warmup, sample_batch, threads):
    """samples/s of the compiled reference on `sample_batch` rows of the workload"""
    from myea_b200 import workloads
    from oracle import ref
    if not ref.available():
        return None
    wl = workloads.BUILDERS[wl_name](batch=sample_batch)
    net = ref.RefNet(wl.desc, wl.opt, threads=threads)
    wl.materialize(net)
    X, Y = wl.batch()
    ms = net.time_steps(X, Y, warmup, steps)
    used = net.threads
    net.close()
    return {"value": sample_batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "cores": used}


def run_reference(args):
    from myea_b200 import workloads
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = min(os.cpu_count() or 1, 32)
    sample = CPU_SAMPLE_ROWS[args.workload]
    steps = max(1, min(args.steps, 3))
    warm = 1 if args.warmup > 0 else 0
    r = cpu_reference_run(args.workload, steps, warm, sample, threads)
    wl = workloads.BUILDERS[args.workload]()
    if r is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libmyea_ref.so was not built (no reference checkout at build time)"}))
        return
    line = {"impl": "reference", "metric": "train samples/sec (fwd+bwd+update)", "value": r["value"], "unit": "samples/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl.name, "global_batch": wl.B, "sample_batch": sample},
            "cpu_baseline": {"value": r["value"], "unit": "samples/s", "cores": r["cores"], "kind": "reference",
                             "sample": "%d rows of the workload per step, %d timed steps, reference OpenMP path" % (sample, steps)},
            "e2e": {"value": r["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


class Job:
    """one network on this rank's GPU for its shard of a global batch, joined to the other ranks when there are any"""

    def __init__(self, torch, dist, workload, per_gpu_batch, world, rank, local, scale=None, opt=None, **kw):
        from myea_b200 import workloads
        from myea_b200.net import Net
        self.torch, self.dist, self.world, self.rank = torch, dist, world, rank
        build = workloads.BUILDERS[workload]
        self.wl = build(batch=per_gpu_batch, **kw) if scale is None else build(scale=scale, batch=per_gpu_batch, **kw)
        if opt is not None:
            self.wl.opt = opt
        self.global_batch = per_gpu_batch * world
        self.net = Net(self.wl.desc, self.wl.opt, device=local)
        self.wl.materialize(self.net)
        self.lib = self.net.lib
        if world > 1:
            uid = torch.zeros(128, dtype=torch.uint8)
            if rank == 0:
                buf = (C.c_uint8 * 128)()
                if self.lib.myea_b200_comm_unique_id(buf) != 0:
                    raise RuntimeError("comm_unique_id failed")
                uid = torch.tensor(list(buf), dtype=torch.uint8)
            uid = uid.cuda()
            dist.broadcast(uid, 0)
            idb = (C.c_uint8 * 128)(*uid.cpu().tolist())
            self.net._ck(self.lib.myea_b200_comm_init(self.net.h, world, rank, idb), "comm_init")
        # this rank's rows of the global batch (rank r owns rows [r*B, (r+1)*B) of every time step)
        B = self.wl.B
        Xg, Yg = self.wl.batch(rows=self.global_batch)
        self.X = np.ascontiguousarray(Xg[:, rank * B:(rank + 1) * B])
        self.Y = np.ascontiguousarray(Yg[:, rank * B:(rank + 1) * B])
        self.Xg, self.Yg = (Xg, Yg) if rank == 0 else (None, None)
        self.Xh, self.Yh = torch.from_numpy(self.X).pin_memory(), torch.from_numpy(self.Y).pin_memory()
        self.Xd, self.Yd = self.Xh.cuda(), self.Yh.cuda()
        self.stream = torch.cuda.ExternalStream(int(self.lib.myea_b200_stream(self.net.h)))

    def step_device(self):
        lib, h, B, gb = self.lib, self.net.h, self.wl.B, self.global_batch
        rc = lib.myea_b200_forward_device(h, B, self.Xd.data_ptr(), 1)
        rc |= lib.myea_b200_compute_error_device(h, B, self.Yd.data_ptr())
        rc |= lib.myea_b200_backward(h, B)
        rc |= lib.myea_b200_update_derivative_weight(h, B)
        rc |= lib.myea_b200_update_parameter(h, gb, gb, C.byref(self.wl.opt))
        return rc

    def step_host(self):
        lib, h, B, gb = self.lib, self.net.h, self.wl.B, self.global_batch
        rc = lib.myea_b200_reset_loss(h)
        rc |= lib.myea_b200_forward(h, B, self.Xh.data_ptr(), 1)
        rc |= lib.myea_b200_compute_error(h, B, self.Yh.data_ptr())
        rc |= lib.myea_b200_backward(h, B)
        rc |= lib.myea_b200_update_derivative_weight(h, B)
        rc |= lib.myea_b200_update_parameter(h, gb, gb, C.byref(self.wl.opt))
        s, n, a = C.c_double(), C.c_uint64(), C.c_double()
        rc |= lib.myea_b200_get_loss(h, C.byref(s), C.byref(n), C.byref(a))  # device -> host read of the step's loss
        return rc

    def timed(self, fn, steps, warmup):
        """(milliseconds for `steps` steps: device time on the library's stream, max over ranks; launches)"""
        torch, dist, net = self.torch, self.dist, self.net
        for _ in range(warmup):
            if fn() != 0:
                raise RuntimeError("step failed: " + self.lib.myea_b200_last_error(net.h).decode())
        net.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = net.launches()
        rc = 0
        e0.record(self.stream)
        for _ in range(steps):
            rc |= fn()
        e1.record(self.stream)
        e1.synchronize()
        torch.cuda.synchronize()
        if rc != 0:   # a step that failed on the host side would otherwise count as a very fast one
            raise RuntimeError("a timed step failed: " + self.lib.myea_b200_last_error(net.h).decode())
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.barrier()
            ms = float(t.item())
        net.synchronize()   # raises when a kernel gave up a bounded wait
        return ms, net.launches() - l0

    def classes(self, steps):
        """per-class device time of `steps` steps (events around every launch: the steps run serialised)"""
        net = self.net
        net.profile(True)
        net.profile_read(reset=True)
        for _ in range(steps):
            self.step_device()
        net.synchronize()
        cls_ms, cls_n, gemm_flops = net.profile_read(reset=True)
        net.profile(False)
        return cls_ms, gemm_flops

    def close(self):
        self.net.close()


def dp_check(torch, dist, world, rank, local, timed_job):
    """correctness of the data-parallel path, on every run with more than one rank:
    (1) the parameter buffers of the timed job are identical on all ranks after the timed steps (bitwise: every rank
        applied the same update to the same sums), (2) two steps of a small network sharded over the ranks equal the same
        two steps on ONE rank with the whole batch, within the parity tolerance.  The small network is updated by momentum
        descent, which is linear in the derivatives: under Adam the first steps are lr * sign(g), and a derivative that is
        zero up to the rounding of its sum takes either sign depending on the order of the sum (seen at 8 ranks: one
        element of 0.4 million off by 2 * lr, everything else equal to 1e-6)"""
    from myea_b200 import capi
    p = torch.from_numpy(timed_job.net.get(capi.BUF_PARAMETERS)).cuda()
    hi, lo = p.clone(), p.clone()
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    spread = float((hi - lo).abs().max().item())
    del p, hi, lo
    linear = capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9)
    small = Job(torch, dist, "c2", 64, world, rank, local, scale=1.0 / 16, opt=linear, hidden_layers=3)
    for _ in range(2):
        if small.step_host() != 0:
            raise RuntimeError("dp_check step failed")
    small.net.synchronize()
    got = small.net.get(capi.BUF_PARAMETERS)
    out = {"parameter_spread_across_ranks": spread,
           # whether the batch-norm column sums travel through the library's own peer-memory exchange kernel (1) or NCCL (0)
           "peer_memory_sums": int(C.CDLL(capi.LIB_PATH).myea_b200_comm_peer_sums(timed_job.net.h)),
           "peer_memory_copies": int(C.CDLL(capi.LIB_PATH).myea_b200_comm_peer_copies(timed_job.net.h))}
    if rank == 0:
        from myea_b200 import workloads
        from myea_b200.net import Net
        wl = workloads.c2_wide_mlp(scale=1.0 / 16, batch=64 * world, hidden_layers=3)
        wl.opt = linear
        one = Net(wl.desc, wl.opt, device=local)
        wl.materialize(one)
        for _ in range(2):
            one.reset_loss(); one.forward(small.Xg); one.compute_error(small.Yg); one.backward(); one.update_derivative_weight(); one.update_parameter()
        want = one.get(capi.BUF_PARAMETERS)
        one.close()
        out["sharded_vs_one_rank_rel_err"] = float(np.abs(got - want).max() / np.abs(want).max())
        out["network"] = "C2 at 1/16 width, 3 hidden layers, momentum descent, global batch %d, 2 steps" % (64 * world)
    small.close()
    return out


def run_ours(args):
    import torch
    from myea_b200 import workloads
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus %d needs torchrun with %d ranks" % (args.gpus, args.gpus))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    full = workloads.BUILDERS[args.workload]()
    global_batch = args.global_batch or full.B
    if global_batch % world != 0:
        raise SystemExit("the global batch %d does not divide over %d ranks" % (global_batch, world))
    kw = {"hidden_layers": args.hidden_layers} if args.hidden_layers else {}
    job = Job(torch, dist, args.workload, global_batch // world, world, rank, local, **kw)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_dev, launches = job.timed(job.step_device, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e, _ = job.timed(job.step_host, args.steps, max(1, args.warmup // 2))
    cls_steps = max(1, min(args.steps, 3))
    cls_ms, gemm_flops = job.classes(cls_steps)
    check = dp_check(torch, dist, world, rank, local, job) if world > 1 else None
    wl = job.wl
    X_bytes, Y_bytes = int(job.X.nbytes), int(job.Y.nbytes)
    job.close()
    del job
    weak = None
    if world > 1 and not args.no_extra:
        # the same step with the configuration's batch on EVERY GPU (weak scaling), for comparison
        wjob = Job(torch, dist, args.workload, full.B, world, rank, local, **kw)
        wms, _ = wjob.timed(wjob.step_device, args.steps, args.warmup)
        weak = {"value": wjob.global_batch / (wms / args.steps / 1e3), "unit": "samples/s", "ms_per_step": wms / args.steps,
                "global_batch": wjob.global_batch, "per_gpu_batch": full.B, "scaling": "weak"}
        wjob.close()
        del wjob
    others = {}
    if world == 1 and args.workload == "c2" and not args.no_extra:
        # the recurrent configuration the throughput target also names, timed after the headline workload
        for name, steps in (("c3", max(3, min(args.steps, 10))),):
            oj = Job(torch, dist, name, workloads.BUILDERS[name]().B, 1, 0, local)
            oms, ol = oj.timed(oj.step_device, steps, 3)
            oe2e, _ = oj.timed(oj.step_host, steps, 1)
            ocls, oflops = oj.classes(2)
            others[name] = {"workload": oj.wl.name, "global_batch": oj.global_batch, "steps": steps, "ms_per_step": oms / steps,
                            "value": oj.global_batch / (oms / steps / 1e3), "unit": "samples/s",
                            "e2e": {"value": oj.global_batch / (oe2e / steps / 1e3), "unit": "samples/s"},
                            "gpu_launches": int(ol), "step_tflops": oj.wl.flops_per_step / (oms / steps / 1e3) / 1e12,
                            "kernel_classes_ms_per_step": {n: m / 2 for n, m in zip(CLASS_NAMES, ocls) if m > 0}}
            oj.close()
            del oj
    peaks = _peaks()
    if rank == 0:
        per_step = ms_dev / args.steps
        value = global_batch / (per_step / 1e3)
        e2e_value = global_batch / ((ms_e2e / args.steps) / 1e3)
        gemm_tflops = gemm_flops / (cls_ms[0] / 1e3) / 1e12 if cls_ms[0] > 0 else 0.0
        peak, burst = peaks["bf16_tflops_sustained"], peaks["bf16_tflops"]
        line = {
            "metric": "train samples/sec (fwd+bwd+update)", "value": value, "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "f32 (split-precision tensor-core products: TF32 hi*hi + BF16 cross terms, fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": wl.name, "global_batch": global_batch, "per_gpu_batch": wl.B,
                       "parallelism": "dp%d" % world, "l2": "per-step working set (> 6 GB at one GPU) far exceeds the 126 MB L2"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": (X_bytes + Y_bytes) * world,
                    "d2h_bytes_per_step": 24 * world},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "achieved": gemm_tflops, "peak": peak, "unit": "TFLOP/s",
                         "frac": gemm_tflops / peak if peak else None,
                         # DRAM bytes of ONE launch of the dominant kernel on the 4096^3 contraction of this workload
                         # (dram__bytes_read.sum + dram__bytes_write.sum of the ncu capture summarised under profiles/;
                         # algorithmic: 335 MB)
                         "traffic": 704.7e6 if args.workload == "c2" else None,
                         "traffic_source": "profiles/gemm3x_tf32_tcgen05_wide_4096x4096x4096.md" if args.workload == "c2" else None,
                         "kernel": "gemm3x_tf32_tcgen05_wide_kernel", "peak_source": peaks["source"] + " bf16 sustained",
                         # every fp32 product costs one TF32 and one BF16 K=16 instruction of equal duration: the
                         # scheme's own ceiling is a quarter of the bf16 peak (sustained: inside a step; burst: alone)
                         "scheme_ceiling": peak / 4.0, "frac_of_scheme_ceiling": gemm_tflops / (peak / 4.0),
                         "scheme_ceiling_burst": burst / 4.0, "frac_of_scheme_ceiling_burst": gemm_tflops / (burst / 4.0),
                         "step_tflops": wl.flops_per_step * world / (per_step / 1e3) / 1e12},
            "kernel_classes_ms_per_step": {n: m / cls_steps for n, m in zip(CLASS_NAMES, cls_ms) if m > 0},
        }
        if check is not None:
            line["dp_check"] = check
        if weak is not None:
            line["weak_scaling"] = weak
        if others:
            line["other_workloads"] = others
        if world == 1 and not args.no_cpu:
            try:
                threads = min(os.cpu_count() or 1, 32)
                sample = CPU_SAMPLE_ROWS[args.workload]
                r = cpu_reference_run(args.workload, 3, 1, sample, threads)
                if r is not None:
                    line["cpu_baseline"] = {"value": r["value"], "unit": "samples/s", "cores": r["cores"], "kind": "reference",
                                            "sample": "%d rows of the workload per step, 3 timed steps after 1 warm-up, reference OpenMP path" % sample}
            except Exception as exc:  # the baseline is reported, never required for the GPU number
                line["cpu_baseline"] = {"value": None, "unit": "samples/s", "cores": 0, "kind": "reference", "sample": "failed: %s" % exc}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def run_gemm(args):
    """one contraction C = A B^T through myea_b200_gemm_nt: error against a float64 product and, with --steps, timing"""
    from myea_b200 import capi
    M, N, K = args.gemm
    lib = capi.load()
    rng = np.random.default_rng(0)
    A = rng.standard_normal((M, K), dtype=np.float32)
    B = rng.standard_normal((N, K), dtype=np.float32)
    out = np.zeros((M, N), np.float32)
    ms = C.c_float(0)
    rc = lib.myea_b200_gemm_nt(0, args.engine, M, N, K, A.ctypes.data, B.ctypes.data, out.ctypes.data, 0, C.byref(ms), args.steps)
    if rc != 0:
        raise SystemExit("myea_b200_gemm_nt failed with status %d" % rc)
    line = {"gemm": [M, N, K], "engine_flags": args.engine}
    if M * N * K <= 2 ** 37:
        want = A.astype(np.float64) @ B.astype(np.float64).T
        line["max_error_over_max_abs"] = float(np.abs(out - want).max() / np.abs(want).max())
    if args.steps > 0:
        line["ms_per_contraction_with_operand_splits"] = ms.value
        line["tflops"] = 2.0 * M * N * K / (ms.value * 1e-3) / 1e12
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--global-batch", type=int, default=None, help="override the configuration's global batch")
    ap.add_argument("--hidden-layers", type=int, default=None, help="c2 only: fewer hidden layers (small captures for profiling)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the weak-scaling and other-workload legs")
    ap.add_argument("--gemm", type=int, nargs=3, metavar=("M", "N", "K"), default=None)
    ap.add_argument("--engine", type=int, default=0, help="--gemm only: engine / tile flags of myea_b200_gemm_nt")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    if args.gemm is not None:
        run_gemm(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
