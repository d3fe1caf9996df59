"""Headline benchmark: the Llama-3-8B decode layer set through the int4 weight-only linear.

One step = one pass of x[M,K] through the four quantized layers of a decoder block
(qkv 6144x4096, o 4096x4096, gate_up 28672x4096, down 4096x14336; int4, tensor_core_tiled layout,
group size 64, M=1 by default).  Weights are synthetic: W ~ N(0, 0.02) in bf16 with 0.1 % of the entries
scaled x20, quantised on the device by this library.  The metric is algorithmic bytes per second:
N*K/2 + (K/g)*N*4 + M*K*2 + M*N*2 bytes per layer, divided by device time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--m M] [--group G]

N > 1 is launched by torch.distributed.run, one rank per GPU.  Every rank then holds the layer set as its
row shard (rank r owns output rows [r*N, (r+1)*N) of layers p times as tall), computes its slice of every
output and all ranks exchange the slices with an all-gather per layer (NCCL over NVLink): per-GPU work is
fixed, so the scaling is weak.

`--impl reference` times the CPU route of the reference for the same workload (dequantise the whole weight
to bf16, then a dense matmul) with the C restatement under oracle/ on all host cores; no GPU is touched.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYERS = [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)]
SEED = 1234
METRIC = "int4 weight-only linear algorithmic GB/s, Llama-3-8B decode layer set (tinygemm layout)"


def algorithmic_bytes(M, N, K, g):
    return N * K // 2 + (K // g) * N * 4 + M * K * 2 + M * N * 2


def step_bytes(M, g):
    return sum(algorithmic_bytes(M, N, K, g) for _, N, K in LAYERS)


def make_weight_cpu(N, K, seed):
    """bf16 W ~ N(0, 0.02) with 0.1 % of the entries multiplied by 20 (CPU generator: same bits everywhere)."""
    gen = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=gen) * 0.02
    mask = torch.rand(N, K, generator=gen) < 0.001
    return torch.where(mask, w * 20, w).to(torch.bfloat16)


def make_x_cpu(M, K, seed):
    gen = torch.Generator().manual_seed(seed)
    return torch.randn(M, K, generator=gen).to(torch.bfloat16)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ----------------------------------------------------------------------------------------------
# clocks: nvidia-smi sampled in a child process during the timed region (read-only query)
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.out = None

    def start(self):
        try:
            self.out = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"], stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.flush()
        self.out.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.out.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(self.NAMES, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.out.close()
        os.unlink(self.out.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
# CPU arm: the reference's CPU route (dequantize_affine to bf16, then a dense linear) restated in C
# ----------------------------------------------------------------------------------------------
class CpuLayerSet:
    """The workload quantised and run on the host by the oracle (never used by the GPU arm's product path)."""

    def __init__(self, M, g, row_fraction=1.0):
        from oracle import oracle as orc
        self.orc, self.M, self.g = orc, M, g
        self.layers = []
        for i, (name, N, K) in enumerate(LAYERS):
            n = max(8, int(N * row_fraction) // 8 * 8)
            w = make_weight_cpu(N, K, SEED + i)[:n].float().numpy()
            s, z = orc.choose_qparams_affine(w, orc.BF16, orc.ASYMMETRIC, [1, g], 0, 15, 1e-6, orc.BF16, orc.BF16, False,
                                             orc.ZP_FLOAT)
            q = orc.quantize_affine(w, orc.BF16, [1, g], s, orc.BF16, z, orc.BF16, 0, 15, orc.ZP_FLOAT).astype(np.uint8)
            x = make_x_cpu(M, K, SEED + 100 + i).float().numpy()
            self.layers.append((name, n, K, q, s, z, x))
        self.wbuf = np.empty(max(n * K for _, n, K, *_ in self.layers), np.float32)
        self.bytes = sum(algorithmic_bytes(M, n, K, g) for _, n, K, *_ in self.layers)

    def step(self):
        out = []
        for _, n, K, q, s, z, x in self.layers:
            out.append(self.orc.int4_linear_dequant_then_matmul(x, q, s, z, self.g, self.wbuf[:n * K].reshape(n, K)))
        return out


def time_cpu(M, g, steps, warmup, row_fraction=1.0):
    cpu = CpuLayerSet(M, g, row_fraction)
    for _ in range(warmup):
        cpu.step()
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu.step()
    dt = (time.perf_counter() - t0) / steps
    sample = "full layer set per step" if row_fraction == 1.0 else f"first {row_fraction:.3f} of every layer's rows per step"
    return {"value": cpu.bytes / dt / 1e9, "unit": "GB/s", "cores": cpu.orc.num_threads(), "kind": "port",
            "sample": f"{sample}, {steps} steps after {warmup} warm-up, {dt * 1e3:.1f} ms/step"}, dt


def run_reference(args):
    """The reference arm: the same config, metric and unit, computed by the CPU route on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, dt = time_cpu(args.m, args.group, args.steps, max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, 1),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, world):
    return {"workload": "llama3-8b decode layer set, int4 weight-only, tensor_core_tiled (inner_k_tiles 8)",
            "layers_NxK": {n: [N, K] for n, N, K in LAYERS}, "M": args.m, "group_size": args.group,
            "weights": "bf16 N(0,0.02), 0.1% entries x20, quantised on device",
            "l2": f"{args.copies} distinct copies of the layer set rotate ({args.copies} x 117 MB > 2 x L2)",
            "parallelism": "single GPU" if world == 1 else
            f"row shards on {world} GPUs, outputs of every layer gathered on every rank "
            f"({'stores over peer memory in the GEMV epilogue' if args.exchange == 'fused' and args.m <= 8 else 'NCCL all-gather'}; "
            "the end-to-end leg goes through RowShardedLinear with the same exchange)"}


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
class GpuLayerSet:
    """`copies` distinct quantised instances of the layer set on one GPU, built through the public API
    (quantize(model, int4_weight_only(g))), plus fixed activation / output / scratch buffers."""

    def __init__(self, M, g, copies, device, rank):
        from ao_b200 import ops
        from ao_b200.quantization import int4_weight_only, quantize
        self.ops, self.M, self.g, self.device = ops, M, g, device
        model = torch.nn.ModuleDict()
        for i, (name, N, K) in enumerate(LAYERS):
            lin = torch.nn.Linear(K, N, bias=False, device=device, dtype=torch.bfloat16)
            with torch.no_grad():
                lin.weight.copy_(make_weight_cpu(N, K, SEED + i + 1000 * rank))
            model[name] = lin
        quantize(model, int4_weight_only(group_size=g, inner_k_tiles=8))
        self.models = [model]
        for _ in range(copies - 1):
            clone = torch.nn.ModuleDict()
            for name, N, K in LAYERS:
                lin = torch.nn.Linear(K, N, bias=False, device="meta", dtype=torch.bfloat16)
                lin.weight = torch.nn.Parameter(model[name].weight.clone(), requires_grad=False)
                clone[name] = lin
            self.models.append(clone)
        # one pinned staging buffer for the step's activations and one for its results (a single copy each way per
        # step); per-layer tensors are views
        def carve(flat, shapes):
            views, off = [], 0
            for r, c in shapes:
                views.append(flat[off:off + r * c].view(r, c))
                off += (r * c + 127) // 128 * 128   # keep every view 256-byte aligned
            return views
        x_shapes = [(M, K) for _, N, K in LAYERS]
        y_shapes = [(M, N) for _, N, K in LAYERS]
        total = lambda shapes: sum((r * c + 127) // 128 * 128 for r, c in shapes)
        self.x_host_all = torch.empty(total(x_shapes), dtype=torch.bfloat16).pin_memory()
        self.x_all = torch.empty(total(x_shapes), dtype=torch.bfloat16, device=device)
        self.y_host_all = torch.empty(total(y_shapes), dtype=torch.bfloat16).pin_memory()
        self.y_all = torch.empty(total(y_shapes), dtype=torch.bfloat16, device=device)
        self.x_host, self.x = carve(self.x_host_all, x_shapes), carve(self.x_all, x_shapes)
        self.y_host, self.y = carve(self.y_host_all, y_shapes), carve(self.y_all, y_shapes)
        for i, (_, N, K) in enumerate(LAYERS):
            self.x_host[i].copy_(make_x_cpu(M, K, SEED + 100 + i))
        self.x_all.copy_(self.x_host_all)
        nbytes = max(ops.int4_workspace_bytes(M, N, K, g, 8) for _, N, K in LAYERS)
        if nbytes <= 0:
            raise RuntimeError("the int4 linear does not support this workload")
        self.ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.launches_per_step = len(LAYERS) * ((M + 15) // 16)
        self.slot_offsets = []
        self.sharded = None

    def use_exchange(self, exchange, world):
        """Public-API form of the sharded step: RowShardedLinear modules whose forward runs the fused exchange."""
        from ao_b200.sharding import RowShardedLinear
        self.sharded = []
        for model in self.models:
            mods = {}
            for i, (name, N, K) in enumerate(LAYERS):
                mods[name] = RowShardedLinear(model[name], N * world, 8, None, exchange, self.slot_offsets[i])
            self.sharded.append(mods)

    def exchange_bytes(self, world):
        """Carves one gathered-output slot per layer in a PeerExchange payload; returns the payload size."""
        off = 0
        self.slot_offsets = []
        for _, N, K in LAYERS:
            self.slot_offsets.append(off)
            off += self.ops.gather_slot_bytes(world, self.M, N)
        return off

    def kernels_only(self, copy, gather=None, exchange=None):
        """The hot path alone: one kernel per layer on resident inputs; sharded runs exchange the outputs per layer,
        in the kernel's epilogue (exchange) or with a collective after it (gather)."""
        model = self.models[copy]
        for i, (name, N, K) in enumerate(LAYERS):
            lt = model[name].weight.layout_tensor
            if exchange is not None:
                self.ops.weight_int4pack_mm_gather(self.x[i], lt.packed_weight, self.g, lt.scale_and_zero, exchange,
                                                   slot_offset_bytes=self.slot_offsets[i], workspace=self.ws)
                continue
            self.ops.weight_int4pack_mm(self.x[i], lt.packed_weight, self.g, lt.scale_and_zero, out=self.y[i],
                                        workspace=self.ws)
            if gather is not None:
                gather(i, self.y[i])

    def end_to_end_enqueue(self, copy, gather=None):
        """What a user runs per decode step: host activations in, module(x) on the quantized modules, results out."""
        model = self.models[copy]
        self.x_all.copy_(self.x_host_all, non_blocking=True)
        for i, (name, N, K) in enumerate(LAYERS):
            if self.sharded is not None:
                y = self.sharded[copy][name](self.x[i])[..., :N]   # full-width output; keep this rank's N columns' worth
            else:
                y = model[name](self.x[i])
                if gather is not None:
                    gather(i, y)
            self.y[i].copy_(y)
        self.y_host_all.copy_(self.y_all, non_blocking=True)

    def end_to_end(self, copy, gather=None):
        self.end_to_end_enqueue(copy, gather)
        torch.cuda.current_stream().synchronize()

    def status(self):
        return int(self.ws[:4].view(torch.int32).item())


def _note(msg):
    """Progress line on stderr (BENCH_VERBOSE=1): where a multi-rank run is when something stalls."""
    if os.environ.get("BENCH_VERBOSE"):
        print(f"[bench rank {os.environ.get('RANK', '0')} +{time.perf_counter() - _T0:.1f}s] {msg}", file=sys.stderr, flush=True)


_T0 = time.perf_counter()


def run_ours(args):
    import torch.distributed as dist
    from ao_b200 import _cabi
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (sm_100a); there is no CPU fallback. "
                           "Use --impl reference for the CPU arm.")
    _cabi.lib()  # fail now if the library has not been built
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=90))
    M, g, copies = args.m, args.group, args.copies
    _note("process group ready; building the layer set")
    ls = GpuLayerSet(M, g, copies, device, rank)
    _note("layer set ready")

    gather, exchange = None, None
    if world > 1:
        gathered = [torch.empty(world, M, N, dtype=torch.bfloat16, device=device) for _, N, K in LAYERS]

        def gather(i, y):
            dist.all_gather_into_tensor(gathered[i], y)

        if args.exchange == "fused" and M <= 8:
            from ao_b200.comm import PeerExchange
            exchange = PeerExchange(ls.exchange_bytes(world))
            ls.use_exchange(exchange, world)
            _note("peer buffers mapped")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # warm up eagerly (module load, attribute set-up, NCCL channels), then capture one graph per copy
    for c in range(copies):
        ls.kernels_only(c, gather, exchange)
    torch.cuda.synchronize()
    _note("eager warm-up done")
    graphs = None
    if not args.no_graph:
        try:
            graphs = []
            for c in range(copies):
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    ls.kernels_only(c, gather, exchange)
                graphs.append(gr)
        except Exception as e:  # capture of the collective can be refused; time plain launches then
            print(f"[bench] CUDA graph capture failed ({type(e).__name__}: {e}); timing plain launches", file=sys.stderr)
            graphs = None
            torch.cuda.synchronize()

    def one_step(i):
        if graphs is not None:
            graphs[i % copies].replay()
        else:
            ls.kernels_only(i % copies, gather)

    _note(f"graphs captured: {graphs is not None}")
    for i in range(max(args.warmup, 3)):
        one_step(i)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # the clock sampler needs a few periods inside the timed region: repeat short regions and keep them all
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for i in range(args.steps):
        one_step(i)
    stop.record()
    barrier()
    ms = start.elapsed_time(stop)
    _note(f"timed region done: {ms:.3f} ms")
    # keep the GPU under the same load a little longer so that nvidia-smi sees it (not part of the number); a fixed
    # count, so that every rank issues the same collectives
    for i in range(6000):
        one_step(i)
        if i % 500 == 499:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    _note("load loop done")
    clocks = sampler.stop() if rank == 0 else None
    if ls.status() != 0:
        raise RuntimeError(f"kernel status word {ls.status()} (a bounded wait ran out)")

    # end to end through the public API with host buffers: eagerly, and with the same step (pinned-host copies in,
    # module calls, copies out) captured once per weight copy in a CUDA graph and replayed, one synchronise per step
    for i in range(max(args.warmup, 3)):
        ls.end_to_end(i % copies, gather)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        ls.end_to_end(i % copies, gather)
    torch.cuda.synchronize()
    e2e_eager_s = time.perf_counter() - t0
    barrier()
    e2e_s, e2e_graph = e2e_eager_s, False
    if graphs is not None:
        try:
            e2e_graphs = []
            for c in range(copies):
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    ls.end_to_end_enqueue(c, gather)
                e2e_graphs.append(gr)
            for i in range(max(args.warmup, 3)):
                e2e_graphs[i % copies].replay()
                torch.cuda.current_stream().synchronize()
            barrier()
            t0 = time.perf_counter()
            for i in range(args.steps):
                e2e_graphs[i % copies].replay()
                torch.cuda.current_stream().synchronize()
            e2e_s = time.perf_counter() - t0
            e2e_graph = True
            barrier()
        except Exception as e:
            print(f"[bench] end-to-end graph capture failed ({type(e).__name__}: {e}); reporting the eager run",
                  file=sys.stderr)
            torch.cuda.synchronize()
    _note("end-to-end region done")

    times = torch.tensor([ms, e2e_s * 1e3, e2e_eager_s * 1e3], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, e2e_eager_ms = float(times[0]), float(times[1]), float(times[2])

    if rank == 0:
        per_rank = step_bytes(M, g)
        total = per_rank * world
        value = total * args.steps / (ms * 1e-3) / 1e9
        e2e_value = total * args.steps / (e2e_ms * 1e-3) / 1e9
        peak, peak_kind = peaks()
        launches = ls.launches_per_step * args.steps
        # dominant kernel: int4_gemv_kernel (every launch of the step); average launch = step time / launches,
        # launch gaps included
        kernel_s = (ms * 1e-3) / launches
        achieved = per_rank / ls.launches_per_step / kernel_s / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args, world),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH.get((M, g)), "peak_kind": f"of {peak_kind}",
                         "kernel": "int4_gemv_kernel", "algorithmic_bytes_per_launch": per_rank / ls.launches_per_step,
                         "avg_launch_us": kernel_s * 1e6},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": ls.x_host_all.numel() * 2,
                    "d2h_bytes_per_step": ls.y_host_all.numel() * 2, "ms_per_step": e2e_ms / args.steps,
                    "mode": "CUDA-graph replay of the public-API step" if e2e_graph else "eager public-API calls",
                    "eager_ms_per_step": e2e_eager_ms / args.steps},
            "gpu_launches": launches,
            "clocks": clocks,
            "graph": graphs is not None,
        }
        if world == 1 and not args.no_cpu_baseline:
            probe, dt = time_cpu(M, g, 1, 1)
            steps = int(min(40, max(3, 8.0 / dt)))
            line["cpu_baseline"], _ = time_cpu(M, g, steps, 1)
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        # orderly shutdown: drop the captured graphs (they reference the communicator's kernels), drain the device,
        # meet at a barrier, then destroy the group; a timer ends the process if the teardown itself stalls (the
        # result line is already out)
        import gc
        import threading
        sys.stdout.flush()
        killer = threading.Timer(10.0, lambda: os._exit(0))
        killer.daemon = True
        killer.start()
        graphs = None
        gc.collect()
        torch.cuda.synchronize()
        if exchange is not None:
            exchange.close()
        dist.barrier()
        torch.cuda.synchronize()
        _note("destroying the process group")
        dist.destroy_process_group()
        _note("process group destroyed")
        killer.cancel()



# ----------------------------------------------------------------------------------------------
# secondary workloads (one kernel family each; used for the profiles, not the headline line)
# ----------------------------------------------------------------------------------------------
def run_secondary(args):
    """--workload fp6_decode | int4_prefill | hqq_prefill | fp6_prefill: one layer shape, rotating weight copies,
    CUDA-graph replay; reports GB/s against the HBM peak (M <= 16) or TFLOP/s against the bf16 tensor peak."""
    from ao_b200 import _cabi, ops
    from ao_b200.prototype.hqq import mixed_mm, pack_hqq_from_rowmajor
    from ao_b200.prototype.quant_llm.quant_llm import to_scaled_tc_fpx
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (sm_100a); there is no CPU fallback.")
    _cabi.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    wl, M, g = args.workload, args.m, args.group
    N, K = (int(v) for v in args.shape.split("x"))
    gen = torch.Generator().manual_seed(SEED)
    wbytes = N * K * 3 // 4 if "fp6" in wl else N * K // 2
    copies = max(1, min(32, int(300e6 // wbytes) + 1)) if M <= 16 else 1   # rotating copies: > 2 x L2 in total
    calls = []
    if wl in ("int4_prefill", "hqq_prefill"):
        w = (torch.randn(N, K, generator=gen) * 0.02).to(torch.bfloat16).to(dev)
        x = torch.randn(M, K, generator=gen).to(torch.bfloat16).to(dev)
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        if wl == "int4_prefill":
            packed, sz = ops.int4_quantize_pack(w, g, 8)
            ws = torch.zeros(max(ops.int4_workspace_bytes(M, N, K, g, 8), 256), dtype=torch.uint8, device=dev)
            calls.append(lambda: ops.weight_int4pack_mm(x, packed, g, sz, out=y, workspace=ws))
            kernel = "umma_linear_kernel<MT, TinygemmPolicy>"
        else:
            s, z, codes = ops.int4_groupwise_quantize(w, g, want_codes=torch.uint8)
            zh = (8.0 - z.float() / s.float()).to(torch.bfloat16).T.contiguous()
            b, sT = pack_hqq_from_rowmajor(codes), s.T.contiguous()
            calls.append(lambda: mixed_mm(x, b, sT, zh, g))
            kernel = "umma_linear_kernel<MT, HqqPolicy>"
        nbytes = N * K // 2 + (K // g) * N * 4 + M * K * 2 + M * N * 2
        dtype = "bf16"
    else:
        w = (torch.randn(N, K, generator=gen) * 0.02).to(torch.float16).to(dev)
        x = torch.randn(M, K, generator=gen).to(torch.float16).to(dev)
        for _ in range(copies):
            packed, scale = to_scaled_tc_fpx(w, 3, 2)
            calls.append(lambda packed=packed, scale=scale: ops.fp6_llm_linear(x, packed, scale))
        kernel = "fp6_gemv_kernel" if M <= 16 else "umma_linear_kernel<MT, Fp6Policy>"
        nbytes = N * K * 3 // 4 + N * 2 + M * K * 2 + M * N * 2
        dtype = "f16"
    for c in calls:
        c()
    torch.cuda.synchronize()
    # one graph = every weight copy once, back to back (as consecutive layers of a model run); a step = one launch
    gr = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(gr, stream=side):
            for c in calls:
                c()
    torch.cuda.current_stream().wait_stream(side)
    graphs = [gr]
    per_replay = len(calls)
    args.steps = max(1, args.steps // per_replay) * per_replay
    for i in range(max(args.warmup, 3)):
        gr.replay()
    sampler = ClockSampler(0)
    sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(args.steps // per_replay):
        gr.replay()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    t_end = time.perf_counter() + 0.4
    while time.perf_counter() < t_end:
        for i in range(50):
            gr.replay()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    sec = ms * 1e-3 / args.steps
    flops = 2.0 * M * N * K
    if M <= 16:
        peak, kind = peaks()
        value, unit = nbytes / sec / 1e9, "GB/s"
        roof = {"bound": "hbm", "achieved": value, "peak": peak, "unit": "GB/s", "frac": value / peak, "traffic": None,
                "peak_kind": f"of {kind}", "kernel": kernel}
    else:
        path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        peak = json.load(open(path))["bf16_tflops"] if os.path.exists(path) else 1590.0
        value, unit = flops / sec / 1e12, "TFLOP/s"
        roof = {"bound": "tensor", "achieved": value, "peak": peak, "unit": "TFLOP/s", "frac": value / peak, "traffic": None,
                "peak_kind": "of measured (burst)" if os.path.exists(path) else "of fallback", "kernel": kernel,
                "gbs": nbytes / sec / 1e9}
    print(json.dumps({
        "metric": f"{wl} {unit}", "value": value, "unit": unit, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype,
        "data": "synthetic", "config": {"workload": wl, "N": N, "K": K, "M": M, "group_size": g if "fp6" not in wl else None,
                                        "l2": f"{per_replay} weight copies rotate" if per_replay > 1 else
                                        "single weight copy (compute-bound shape)"},
        "roofline": roof, "gpu_launches": args.steps, "clocks": clocks, "cpu_baseline": None, "e2e": None}), flush=True)


# DRAM bytes (read + written) per launch of int4_gemv_kernel averaged over the layer set, from the ncu capture
# summarised under profiles/; keyed by (M, group size).  Missing key: not captured.
TRAFFIC_BYTES_PER_LAUNCH = {(1, 64): 30860736}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--m", type=int, default=1, help="activation rows (decode batch)")
    ap.add_argument("--group", type=int, default=64, choices=[32, 64, 128, 256])
    ap.add_argument("--copies", type=int, default=3, help="distinct instances of the weights that rotate (L2)")
    ap.add_argument("--no-graph", action="store_true", help="plain launches instead of CUDA-graph replay")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", choices=["fused", "nccl"], default="fused",
                    help="N > 1: outputs exchanged by the GEMV epilogue over peer memory, or by an NCCL all-gather")
    ap.add_argument("--workload", default="decode_int4",
                    choices=["decode_int4", "fp6_decode", "int4_prefill", "hqq_prefill", "fp6_prefill"],
                    help="decode_int4 is the headline layer set; the others time one layer shape (--shape NxK, --m)")
    ap.add_argument("--shape", default="8192x8192", help="N x K of the secondary workloads")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        if args.steps > 30:
            args.steps = 30  # ~0.1-0.2 s per step on the host
        run_reference(args)
        return
    if args.workload != "decode_int4":
        run_secondary(args)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (launch with torch.distributed.run); got {world}")
    run_ours(args)


if __name__ == "__main__":
    main()
