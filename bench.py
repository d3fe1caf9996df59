"""Headline benchmark: the Llama-3-8B decode layer set through the int4 weight-only linear.

One step = one pass of x[M,K] through the four quantized layers of a decoder block
(qkv 6144x4096, o 4096x4096, gate_up 28672x4096, down 4096x14336; int4, tensor_core_tiled layout,
group size 64, M=1 by default).  Weights are synthetic: W ~ N(0, 0.02) in bf16 with 0.1 % of the entries
scaled x20, quantised on the device by this library.  The metric is algorithmic bytes per second:
N*K/2 + (K/g)*N*4 + M*K*2 + M*N*2 bytes per layer, divided by device time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--m M] [--group G]

N > 1 is launched by torch.distributed.run, one rank per GPU.  Every rank then holds the layer set as its
row shard (rank r owns output rows [r*N, (r+1)*N) of layers p times as tall) and computes its slice of every output;
the slices are exchanged over NVLink: for M <= 8 one small kernel per step stores the slices of all four layers into
every peer's memory and collects what the peers sent (the four layers of the step take independent inputs, so nothing
needs a layer's gathered output before the step ends); otherwise an NCCL all-gather follows every layer.  Per-GPU work is
fixed, so the scaling is weak.

The same JSON line carries, for the record of the other configurations: `secondary` (1 GPU: FP6 decode, the HQQ-layout
and tensor_core_tiled prefill GEMMs, the FP6 prefill GEMM, each with its own roofline), `config5` (every N: the
Llama-3-70B layer set, group 128, row-sharded with strong scaling, M in {1, 32, 256}) and `kernel_to_beat` (1 GPU:
PyTorch's own aten::_weight_int4pack_mm on the same packed operands, timed the same way).

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
LAYERS_70B = [("qkv", 10240, 8192), ("o", 8192, 8192), ("gate_up", 57344, 8192), ("down", 8192, 28672)]
SEED = 1234
METRIC = "int4 weight-only linear algorithmic GB/s, Llama-3-8B decode layer set (tinygemm layout)"


def algorithmic_bytes(M, N, K, g):
    return N * K // 2 + (K // g) * N * 4 + M * K * 2 + M * N * 2


def step_bytes(M, g, layers=LAYERS):
    return sum(algorithmic_bytes(M, N, K, g) for _, N, K in layers)


def make_weight_cpu(N, K, seed):
    """bf16 W ~ N(0, 0.02) with 0.1 % of the entries multiplied by 20 (CPU generator: same bits everywhere)."""
    gen = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=gen) * 0.02
    mask = torch.rand(N, K, generator=gen) < 0.001
    return torch.where(mask, w * 20, w).to(torch.bfloat16)


def make_x_cpu(M, K, seed):
    gen = torch.Generator().manual_seed(seed)
    return torch.randn(M, K, generator=gen).to(torch.bfloat16)


def measured_peaks():
    """(HBM GB/s, dense bf16 TFLOP/s burst, kind): the driver's measurements on this pool, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


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


def time_regions(run_region, regions, barrier):
    """Times `regions` repetitions of run_region() with CUDA events on the current stream, each bracketed by
    barrier() (a process-group barrier when there is one, and a device synchronise); returns the list of ms."""
    out = []
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(regions):
        barrier()
        start.record()
        run_region()
        stop.record()
        barrier()
        out.append(start.elapsed_time(stop))
    return out


# ----------------------------------------------------------------------------------------------
# CPU arm: the reference's CPU route (dequantize_affine to bf16, then a dense linear) restated in C
# ----------------------------------------------------------------------------------------------
class CpuLayerSet:
    """The workload quantised and run on the host by the oracle (never used by the GPU arm's product path)."""

    def __init__(self, M, g, row_fraction=1.0):
        from oracle import oracle as orc
        self.orc, self.M, self.g = orc, M, g
        # every core this process may use, whatever OMP_NUM_THREADS the launcher exported for its ranks
        self.cores = orc.set_num_threads(0)
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
    return {"value": cpu.bytes / dt / 1e9, "unit": "GB/s", "cores": cpu.cores, "kind": "port",
            "sample": f"{sample}, {steps} steps after {warmup} warm-up, {dt * 1e3:.1f} ms/step"}, dt


def run_reference(args):
    """The reference arm: the same config, metric and unit, computed by the CPU route on the host cores.  Under a
    multi-rank launch rank 0 alone works (on all host cores) and prints; the other ranks exit."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    base, dt = time_cpu(args.m, args.group, args.steps, max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, max(world, args.gpus)),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, world):
    fused = args.exchange == "fused" and args.m <= 8
    return {"workload": "llama3-8b decode layer set, int4 weight-only, tensor_core_tiled (inner_k_tiles 8)",
            "layers_NxK": {n: [N, K] for n, N, K in LAYERS}, "M": args.m, "group_size": args.group,
            "weights": "bf16 N(0,0.02), 0.1% entries x20, quantised on device",
            "l2": f"{args.copies} distinct copies of the layer set rotate ({args.copies} x 117 MB > 2 x L2)",
            "parallelism": "single GPU" if world == 1 else
            f"row shards on {world} GPUs, outputs of every layer gathered on every rank "
            f"({'one gather-exchange kernel per step: 8-byte tagged stores into peer memory, then a bounded poll' if fused else 'NCCL all-gather per layer'}; "
            "the end-to-end leg goes through RowShardedLinear: GEMV + gather-exchange per layer)"}


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
class GpuLayerSet:
    """`copies` distinct quantised instances of a layer set on one GPU, built through the public API
    (quantize(model, int4_weight_only(g))), plus fixed activation / output / scratch buffers."""

    def __init__(self, M, g, copies, device, rank, layers=LAYERS, device_weights=False):
        from ao_b200 import ops
        from ao_b200.dtypes import use_static_linear_outputs
        from ao_b200.quantization import int4_weight_only, quantize
        self.ops, self.M, self.g, self.device, self.layers = ops, M, g, device, layers
        model = torch.nn.ModuleDict()
        dgen = torch.Generator(device=device).manual_seed(SEED + 7 * rank)
        for i, (name, N, K) in enumerate(layers):
            lin = torch.nn.Linear(K, N, bias=False, device="meta", dtype=torch.bfloat16)
            if device_weights:   # large layer sets: N(0, 0.02) drawn on the device
                w = (torch.randn(N, K, generator=dgen, device=device) * 0.02).to(torch.bfloat16)
            else:
                w = make_weight_cpu(N, K, SEED + i + 1000 * rank).to(device)
            lin.weight = torch.nn.Parameter(w, requires_grad=False)
            model[name] = lin
            quantize(lin, int4_weight_only(group_size=g, inner_k_tiles=8))
            del w
        self.models = [model]
        for _ in range(copies - 1):
            clone = torch.nn.ModuleDict()
            for name, N, K in layers:
                lin = torch.nn.Linear(K, N, bias=False, device="meta", dtype=torch.bfloat16)
                lin.weight = torch.nn.Parameter(model[name].weight.clone(), requires_grad=False)
                clone[name] = lin
            self.models.append(clone)

        # one pinned staging buffer for the step's activations (a single copy in per step); per-layer tensors are views
        def carve(flat, shapes):
            views, off = [], 0
            for r, c in shapes:
                views.append(flat[off:off + r * c].view(r, c))
                off += (r * c + 127) // 128 * 128   # keep every view 256-byte aligned
            return views
        x_shapes = [(M, K) for _, N, K in layers]
        y_shapes = [(M, N) for _, N, K in layers]
        total = lambda shapes: sum((r * c + 127) // 128 * 128 for r, c in shapes)
        self.x_host_all = torch.empty(total(x_shapes), dtype=torch.bfloat16).pin_memory()
        self.x_all = torch.empty(total(x_shapes), dtype=torch.bfloat16, device=device)
        self.y_host_all = torch.empty(total(y_shapes), dtype=torch.bfloat16).pin_memory()
        self.y_all = torch.empty(total(y_shapes), dtype=torch.bfloat16, device=device)
        self.x_host, self.x = carve(self.x_host_all, x_shapes), carve(self.x_all, x_shapes)
        self.y_host, self.y = carve(self.y_host_all, y_shapes), carve(self.y_all, y_shapes)
        # module(x) writes straight into the step's result buffer: no allocation and no device-side copy per token
        for m in self.models:
            use_static_linear_outputs(m, outputs={name: self.y[i] for i, (name, N, K) in enumerate(layers)})
        for i, (_, N, K) in enumerate(layers):
            self.x_host[i].copy_(make_x_cpu(M, K, SEED + 100 + i))
        self.x_all.copy_(self.x_host_all)
        nbytes = max(ops.int4_workspace_bytes(M, N, K, g, 8) for _, N, K in layers)
        if nbytes <= 0:
            raise RuntimeError("the int4 linear does not support this workload")
        self.ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.launches_per_step = len(layers) * ((M + 15) // 16)
        self.sites = None
        self.sharded = None
        self.exchange = None

    def exchange_bytes(self, world):
        return 2 * sum(self.ops.gather_slot_bytes(world, self.M, N) for _, N, K in self.layers)

    def use_exchange(self, exchange, world):
        """Call sites for the kernels-only leg, and the public-API form of the sharded step: RowShardedLinear
        modules (call sites of their own) whose forward runs the GEMV and the gather-exchange."""
        from ao_b200.sharding import RowShardedLinear
        self.exchange = exchange
        self.sites = [exchange.reserve(self.M, N) for _, N, K in self.layers]
        self.sharded = []
        e2e_sites = [exchange.reserve(self.M, N) for _, N, K in self.layers]
        for model in self.models:
            mods = {}
            for i, (name, N, K) in enumerate(self.layers):
                mods[name] = RowShardedLinear(model[name], N * world, 8, None, exchange)
                mods[name]._sites[self.M] = e2e_sites[i]     # the copies run one after the other: they share sites
            self.sharded.append(mods)
        self.launches_per_step += 1   # the gather-exchange kernel

    def kernels_only(self, copy, gather=None):
        """The hot path alone: one kernel per layer on resident inputs.  Sharded runs exchange the outputs: one
        gather-exchange kernel per step sends this rank's rows of all layers to the peers' memory and collects theirs
        (peer-memory exchange), or a collective follows every layer (gather)."""
        model = self.models[copy]
        for i, (name, N, K) in enumerate(self.layers):
            lt = model[name].weight.layout_tensor
            if self.sites is not None:    # this rank's block of the layer's gathered output
                self.ops.weight_int4pack_mm(self.x[i], lt.packed_weight, self.g, lt.scale_and_zero,
                                            out=self.sites[i].y[self.exchange.rank], workspace=self.ws)
                continue
            self.ops.weight_int4pack_mm(self.x[i], lt.packed_weight, self.g, lt.scale_and_zero, out=self.y[i],
                                        workspace=self.ws)
            if gather is not None:
                gather(i, self.y[i])
        if self.sites is not None:
            self.ops.gather_exchange(self.exchange, self.sites, push=True, workspace=self.ws)

    def end_to_end_enqueue(self, copy, gather=None):
        """What a user runs per decode step: host activations in (one copy), module(x) on the quantized modules
        (each writes into its slice of the step's result buffer), results out (one copy)."""
        model = self.models[copy]
        self.x_all.copy_(self.x_host_all, non_blocking=True)
        for i, (name, N, K) in enumerate(self.layers):
            if self.sharded is not None:
                y = self.sharded[copy][name](self.x[i])[..., :N]   # full-width output; keep this rank's N columns' worth
                self.y[i].copy_(y)
            else:
                y = model[name](self.x[i])
                if gather is not None:
                    gather(i, y)
        self.y_host_all.copy_(self.y_all, non_blocking=True)

    def end_to_end(self, copy, gather=None):
        self.end_to_end_enqueue(copy, gather)
        torch.cuda.current_stream().synchronize()

    def status(self):
        return int(self.ws[:4].view(torch.int32).item())

    def release(self):
        """Frees the set's device memory (before the next workload allocates its own)."""
        self.models, self.sharded = [], None
        torch.cuda.empty_cache()


def _note(msg):
    """Progress line on stderr (BENCH_VERBOSE=1): where a multi-rank run is when something stalls."""
    if os.environ.get("BENCH_VERBOSE"):
        print(f"[bench rank {os.environ.get('RANK', '0')} +{time.perf_counter() - _T0:.1f}s] {msg}", file=sys.stderr, flush=True)


_T0 = time.perf_counter()


def check_gathered_outputs(ls, world, rank, dist, what):
    """One-time check outside the timed region: what the fused exchange left in every call site equals the
    all-gather of the ranks' single-GPU results, bit for bit, on every rank.  Aborts the run on a mismatch."""
    ok = True
    model = ls.models[0]
    ls.kernels_only(0)
    torch.cuda.synchronize()
    for i, (name, N, K) in enumerate(ls.layers):
        lt = model[name].weight.layout_tensor
        y_local = ls.ops.weight_int4pack_mm(ls.x[i], lt.packed_weight, ls.g, lt.scale_and_zero)
        ref = torch.empty(world, ls.M, N, dtype=torch.bfloat16, device=ls.device)
        dist.all_gather_into_tensor(ref, y_local)
        if not torch.equal(ref, ls.sites[i].y):
            ok = False
    flag = torch.tensor([0 if ok else 1], device=ls.device)
    dist.all_reduce(flag)
    if int(flag.item()) != 0:
        raise RuntimeError(f"{what}: the fused exchange's gathered outputs differ from all_gather of the single-GPU "
                           f"results on {int(flag.item())} rank(s)")
    if rank == 0:
        print(f"[bench] {what}: gathered outputs of all {len(ls.layers)} layers equal all_gather of the single-GPU "
              f"results on all {world} ranks", file=sys.stderr, flush=True)


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
        # stdout carries the one JSON line: no NCCL version banner on it (NCCL_DEBUG=VERSION prints one to stdout), and
        # NCCL's other messages go to stderr
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
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
        ls.kernels_only(c, gather)
    torch.cuda.synchronize()
    _note("eager warm-up done")
    if exchange is not None:
        check_gathered_outputs(ls, world, rank, dist, "8B decode set")
    graphs = None
    if not args.no_graph:
        try:
            graphs = []
            for c in range(copies):
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    ls.kernels_only(c, gather)
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
    # the timed region (exactly `steps` steps between two barriers) is repeated; the median region is the number
    # of record, min and max are reported beside it, and the clock sampler sees load for the whole time
    regions = args.regions

    def region():
        for i in range(args.steps):
            one_step(i)

    region_ms = time_regions(region, regions, barrier)
    _note(f"timed regions done: median {statistics.median(region_ms):.3f} ms")
    t_end = time.perf_counter() + 0.5    # at least half a second under the same load for the clock samples
    more = torch.tensor([0], device=device)
    while True:
        for i in range(200):
            one_step(i)
        torch.cuda.synchronize()
        more[0] = 1 if time.perf_counter() < t_end else 0
        if world > 1:
            dist.all_reduce(more, op=dist.ReduceOp.MIN)   # every rank leaves the loop in the same round
        if int(more.item()) == 0:
            break
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
    e2e_graphs = None
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
    if ls.status() != 0:
        raise RuntimeError(f"kernel status word {ls.status()} (a bounded wait ran out)")
    _note("end-to-end region done")

    ms_med, ms_min, ms_max = statistics.median(region_ms), min(region_ms), max(region_ms)
    times = torch.tensor([ms_med, e2e_s * 1e3, e2e_eager_s * 1e3, ms_min, ms_max], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, e2e_eager_ms, ms_min, ms_max = (float(v) for v in times)
    launches_per_step, x_bytes, y_bytes = ls.launches_per_step, ls.x_host_all.numel() * 2, ls.y_host_all.numel() * 2

    # the other configurations, for the record (not part of the headline number)
    kernel_to_beat = None
    if world == 1 and not args.headline_only:
        kernel_to_beat = time_kernel_to_beat(ls, args, barrier)
    graphs = e2e_graphs = None
    torch.cuda.synchronize()
    ls.release()
    if exchange is not None:
        exchange.close()
        exchange = None
    config5 = run_config5(args, world, rank, device, dist, barrier) if not args.headline_only else None
    secondary = run_secondary_list(args) if (world == 1 and not args.headline_only) else None

    if rank == 0:
        per_rank = step_bytes(M, g)
        total = per_rank * world
        value = total * args.steps / (ms * 1e-3) / 1e9
        e2e_value = total * args.steps / (e2e_ms * 1e-3) / 1e9
        peak, _, peak_kind = measured_peaks()
        gemv_launches = len(LAYERS) * ((M + 15) // 16)
        # dominant kernel: int4_gemv_kernel (the four GEMV launches of a step); average launch = step time / GEMV
        # launches, launch gaps (and, sharded, the gather-wait kernel) included
        kernel_s = (ms * 1e-3) / (gemv_launches * args.steps)
        achieved = per_rank / gemv_launches / kernel_s / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args, world),
            "timed_regions": {"n": regions, "steps_each": args.steps, "ms_per_step_median": ms / args.steps,
                              "ms_per_step_min": ms_min / args.steps, "ms_per_step_max": ms_max / args.steps,
                              "note": "max over ranks of each statistic; value uses the median region"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH.get((M, g)), "peak_kind": f"of {peak_kind}",
                         "kernel": "int4_gemv_kernel", "algorithmic_bytes_per_launch": per_rank / gemv_launches,
                         "avg_launch_us": kernel_s * 1e6},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": x_bytes,
                    "d2h_bytes_per_step": y_bytes, "ms_per_step": e2e_ms / args.steps,
                    "mode": "CUDA-graph replay of the public-API step" if e2e_graph else "eager public-API calls",
                    "eager_ms_per_step": e2e_eager_ms / args.steps},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "graph": not args.no_graph,
            "kernel_to_beat": kernel_to_beat,
            "config5": config5,
            "secondary": secondary,
        }
        if world == 1 and not args.no_cpu_baseline:
            probe, dt = time_cpu(M, g, 1, 1)
            steps = int(min(40, max(3, 8.0 / dt)))
            line["cpu_baseline"], _ = time_cpu(M, g, steps, 1)
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        # orderly shutdown: drain the device, meet at a barrier, then destroy the group; a timer ends the process if
        # the teardown itself stalls (the result line is already out)
        import gc
        import threading
        sys.stdout.flush()
        killer = threading.Timer(10.0, lambda: os._exit(0))
        killer.daemon = True
        killer.start()
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        _note("destroying the process group")
        dist.destroy_process_group()
        _note("process group destroyed")
        killer.cancel()


# ----------------------------------------------------------------------------------------------
# kernel to beat: PyTorch's own tinygemm operator on the same packed operands, timed the same way
# ----------------------------------------------------------------------------------------------
def time_kernel_to_beat(ls, args, barrier):
    name = "torch.ops.aten._weight_int4pack_mm (PyTorch's tinygemm kernel) on the same packed operands, CUDA-graph replay"
    try:
        outs = [None] * len(LAYERS)

        def step(copy):
            model = ls.models[copy]
            for i, (lname, N, K) in enumerate(LAYERS):
                lt = model[lname].weight.layout_tensor
                outs[i] = torch.ops.aten._weight_int4pack_mm(ls.x[i], lt.packed_weight, ls.g, lt.scale_and_zero)

        for c in range(len(ls.models)):
            step(c)
        torch.cuda.synchronize()
        graphs = []
        for c in range(len(ls.models)):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                step(c)
            graphs.append(gr)
        for i in range(5):
            graphs[i % len(graphs)].replay()
        steps = min(args.steps, 200)

        def region():
            for i in range(steps):
                graphs[i % len(graphs)].replay()

        ms = time_regions(region, 7, barrier)
        med = statistics.median(ms) / steps
        return {"kernel": name, "ms_per_step": med, "value": step_bytes(args.m, args.group) / (med * 1e-3) / 1e9,
                "unit": "GB/s", "steps": steps, "regions": 7}
    except Exception as e:  # noqa: BLE001 - the operator may be missing or reject the operands in this torch build
        torch.cuda.synchronize()
        return {"kernel": name, "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}


# ----------------------------------------------------------------------------------------------
# config 5: Llama-3-70B layer set, group 128, N-sharded (strong scaling), M in {1, 32, 256}
# ----------------------------------------------------------------------------------------------
def run_config5(args, world, rank, device, dist, barrier):
    """Every rank holds rows [r*N/p, (r+1)*N/p) of each 70B layer, quantised on its own device; the outputs are
    gathered on every rank: by one gather-exchange kernel per step at M <= 64, by an NCCL all-gather per layer above.  Enough copies of the shard rotate that the weights of consecutive steps never sit in L2."""
    g = 128
    packed_mb = sum(N * K // 2 for _, N, K in LAYERS_70B) / 1e6
    out = {"workload": "llama3-70b layer set, int4 weight-only, tensor_core_tiled, group 128, rows sharded over "
                       f"{world} GPU(s) (strong scaling: the whole set is {packed_mb:.0f} MB packed)",
           "layers_NxK": {n: [N, K] for n, N, K in LAYERS_70B}, "results": []}
    shard = [(n, N // world, K) for n, N, K in LAYERS_70B]
    shard_bytes = sum(N * K // 2 for _, N, K in shard)
    copies = max(1, -(-300_000_000 // shard_bytes))      # >= 300 MB of distinct weights in rotation
    peak_hbm, peak_tf, kind = measured_peaks()
    for M in (1, 32, 256):
        try:
            res = _config5_one(args, world, rank, device, dist, barrier, shard, copies, g, M)
        except Exception as e:  # noqa: BLE001 - one failing batch size must not lose the headline line
            torch.cuda.synchronize()
            res = {"M": M, "error": f"{type(e).__name__}: {str(e)[:200]}"}
        if "ms_per_step" in res:
            sec = res["ms_per_step"] * 1e-3
            total_bytes = step_bytes(M, g, LAYERS_70B)
            flops = sum(2.0 * M * N * K for _, N, K in LAYERS_70B)
            res.update({"gbs_total": total_bytes / sec / 1e9, "hbm_frac_per_gpu": total_bytes / world / sec / 1e9 / peak_hbm,
                        "tflops_total": flops / sec / 1e12, "tensor_frac_per_gpu": flops / world / sec / 1e12 / peak_tf,
                        "peak_kind": f"of {kind}"})
        out["results"].append(res)
    return out


def _config5_one(args, world, rank, device, dist, barrier, shard, copies, g, M):
    ls = GpuLayerSet(M, g, copies, device, rank, layers=shard, device_weights=True)
    gather, exchange = None, None
    if world > 1:
        gathered = [torch.empty(world, M, N, dtype=torch.bfloat16, device=device) for _, N, K in shard]

        def gather(i, y):
            dist.all_gather_into_tensor(gathered[i], y)

        if M <= 64 and args.exchange == "fused":   # (above that the 8-byte words' factor 2 on the wire outweighs the latency saved)
            from ao_b200.comm import PeerExchange
            exchange = PeerExchange(ls.exchange_bytes(world))
            ls.use_exchange(exchange, world)
    for c in range(copies):
        ls.kernels_only(c, gather)
    torch.cuda.synchronize()
    if exchange is not None:
        check_gathered_outputs(ls, world, rank, dist, f"70B set M={M}")
    graphs = []
    try:
        for c in range(copies):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                ls.kernels_only(c, gather)
            graphs.append(gr)
    except Exception as e:  # noqa: BLE001
        print(f"[bench] config 5 graph capture failed ({type(e).__name__}: {e}); timing plain launches", file=sys.stderr)
        torch.cuda.synchronize()
        graphs = []

    def step(i):
        if graphs:
            graphs[i % copies].replay()
        else:
            ls.kernels_only(i % copies, gather)

    steps = 60 if M == 1 else (40 if M == 32 else 20)
    for i in range(6):
        step(i)

    def region():
        for i in range(steps):
            step(i)

    ms = time_regions(region, 5, barrier)
    t = torch.tensor([statistics.median(ms)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res = {"M": M, "ms_per_step": float(t[0]) / steps, "copies": copies, "steps": steps, "status": ls.status(),
           "exchange": "peer memory (one gather-exchange kernel per step)" if exchange is not None else
           ("NCCL all-gather per layer" if world > 1 else "none")}
    graphs = None
    torch.cuda.synchronize()
    ls.release()
    if exchange is not None:
        exchange.close()
    return res


# ----------------------------------------------------------------------------------------------
# secondary workloads (one kernel family each): --workload X prints one line; the headline run carries a list
# ----------------------------------------------------------------------------------------------
def time_secondary(wl, N, K, M, g, steps, warmup):
    """One layer shape, rotating weight copies (decode shapes), CUDA-graph replay; GB/s against the HBM peak
    (M <= 16) or TFLOP/s against the bf16 tensor peak."""
    from ao_b200 import _cabi, ops
    from ao_b200.prototype.hqq import mixed_mm, pack_hqq_from_rowmajor
    from ao_b200.prototype.quant_llm.quant_llm import to_scaled_tc_fpx
    dev = torch.device("cuda", torch.cuda.current_device())
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
    per_replay = len(calls)
    steps = max(1, steps // per_replay) * per_replay
    for i in range(max(warmup, 3)):
        gr.replay()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(steps // per_replay):
        gr.replay()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    t_end = time.perf_counter() + 0.3
    while time.perf_counter() < t_end:
        for i in range(20):
            gr.replay()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    sec = ms * 1e-3 / steps
    flops = 2.0 * M * N * K
    peak_hbm, peak_tf, kind = measured_peaks()
    if M <= 16:
        value, unit = nbytes / sec / 1e9, "GB/s"
        roof = {"bound": "hbm", "achieved": value, "peak": peak_hbm, "unit": "GB/s", "frac": value / peak_hbm,
                "traffic": None, "peak_kind": f"of {kind}", "kernel": kernel}
    else:
        value, unit = flops / sec / 1e12, "TFLOP/s"
        roof = {"bound": "tensor", "achieved": value, "peak": peak_tf, "unit": "TFLOP/s", "frac": value / peak_tf,
                "traffic": None, "peak_kind": f"of {kind} (burst)", "kernel": kernel, "gbs": nbytes / sec / 1e9}
    status = _cabi.workspace_status(dev)
    del gr, calls
    torch.cuda.empty_cache()
    return {
        "metric": f"{wl} {unit}", "value": value, "unit": unit, "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3),
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype,
        "data": "synthetic", "config": {"workload": wl, "N": N, "K": K, "M": M, "group_size": g if "fp6" not in wl else None,
                                        "l2": f"{per_replay} weight copies rotate" if per_replay > 1 else
                                        "single weight copy (compute-bound shape)"},
        "roofline": roof, "gpu_launches": steps, "clocks": clocks, "status": status, "cpu_baseline": None, "e2e": None}


SECONDARY_LIST = [
    # (workload, N, K, M, group, steps)
    ("fp6_decode", 12288, 4096, 1, 64, 400),
    ("fp6_decode", 4096, 4096, 1, 64, 400),
    ("hqq_prefill", 8192, 8192, 64, 64, 200),
    ("hqq_prefill", 8192, 8192, 256, 64, 200),
    ("hqq_prefill", 8192, 8192, 1024, 64, 100),
    ("hqq_prefill", 8192, 8192, 4096, 64, 50),
    ("int4_prefill", 8192, 8192, 4096, 64, 50),
    ("fp6_prefill", 12288, 4096, 128, 64, 200),
]


def run_secondary_list(args):
    """The other kernel families at their configured shapes, a few seconds each."""
    out = []
    for wl, N, K, M, g, steps in SECONDARY_LIST:
        try:
            r = time_secondary(wl, N, K, M, g, steps, 5)
            out.append({k: r[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "dtype", "config", "roofline",
                                          "clocks", "status")})
        except Exception as e:  # noqa: BLE001 - one failing family must not lose the headline line
            out.append({"config": {"workload": wl, "N": N, "K": K, "M": M}, "error": f"{type(e).__name__}: {str(e)[:200]}"})
            torch.cuda.synchronize()
    return out


def run_secondary(args):
    from ao_b200 import _cabi
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (sm_100a); there is no CPU fallback.")
    _cabi.lib()
    torch.cuda.set_device(0)
    N, K = (int(v) for v in args.shape.split("x"))
    print(json.dumps(time_secondary(args.workload, N, K, args.m, args.group, args.steps, args.warmup)), flush=True)


# DRAM bytes (read + written) per launch of int4_gemv_kernel averaged over the layer set, from the ncu capture
# summarised under profiles/; keyed by (M, group size).  Missing key: not captured.
TRAFFIC_BYTES_PER_LAUNCH = {(1, 64): 30862208}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--m", type=int, default=1, help="activation rows (decode batch)")
    ap.add_argument("--group", type=int, default=64, choices=[32, 64, 128, 256])
    ap.add_argument("--copies", type=int, default=3, help="distinct instances of the weights that rotate (L2)")
    ap.add_argument("--regions", type=int, default=50, help="repetitions of the timed region (the median counts)")
    ap.add_argument("--no-graph", action="store_true", help="plain launches instead of CUDA-graph replay")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--headline-only", action="store_true", help="skip secondary, config5 and kernel_to_beat")
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
