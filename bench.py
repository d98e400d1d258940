"""bench.py: weight-stream throughput of the dense_reader decode matmul on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c1|c5] [--rows M] [--impl reference]

One step is one pass of the hot path over one batch of synthetic input: one call of linear.matmul. The default
workload ("c2") is the Llama-3-8B MLP gate/up pair, x [1, 4096] bf16, two [14336, 4096] bfloat4_b weights with float32
per-column scales, output silu(x Wg) * (x Wu) in bf16. Inputs are seeded synthetic tensors of those shapes and
distributions (there are no checkpoints here).

Printed: ONE JSON line. `value` is weight-stream GB/s (packed weight bytes of the calls / device time, CUDA events,
max over ranks, all ranks' bytes), inputs resident in HBM, the K steps replayed from one CUDA graph. The weights are
smaller than the 126 MB L2, so the steps rotate over enough distinct packed copies to exceed twice the L2 (`config.l2`).
`e2e` is the same metric through the public Python API with host buffers: every step copies x from pinned host
memory, runs the op and reads y back to pinned host memory (one library call a step, two steps in flight; the
one-step-at-a-time latency is given beside it). `roofline` compares the kernel's algorithmic bytes per launch with the
measured HBM copy bandwidth (the driver's peak file at the repository root, when present). `cpu_baseline` (rank 0,
N = 1) times the reference's torch path (the oracle's port of dense_reader/linear.py:166-169 plus the SwiGLU stage) on
the host cores on a bounded column sample of the same workload, for a fixed wall time.

Beside the headline the line carries, timed in the same run: `sub` (the down projection, bfloat8_b [4096, 14336] with a
float32 residual, one row), `rows32` (the same at 32 rows: the metric is quoted at one row and at 32) and, with N > 1,
`c5_strong` (the LM head's 151936 columns split over the N ranks, top-k records exchanged, global top-32 on every rank).

N > 1 (torchrun, one rank per GPU, NCCL): weak scaling. Each rank streams its own column shard of the same size (a layer
N times as wide, column-sharded as native_weight would pack it per rank) and every rank ends each step holding all
ranks' outputs: by default the stream kernel stores them into the other ranks' buffers itself (peer stores over NVLink,
sharded.Exchange); --exchange nccl all-gathers them with NCCL on a side stream instead. Before anything is timed every
rank checks the exchanged buffer bit for bit against an NCCL all-gather of the ranks' own outputs (`exchange_check`).

--impl reference: the reference's own CPU implementation of the path (the oracle port; the reference's device path needs
ttnn and a Tensix simulator, neither of which exists here), all host threads, same metric.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tensix-kernels_b200"))

import torch  # noqa: E402

WORKLOADS = {
    # name: (K, N per weight, format, description)
    "c1": dict(k=2048, n=4096, fmt="bfp8", what="README example: x[1,2048] @ W[4096,2048] bfloat8_b, no epilogue"),
    "c2": dict(k=4096, n=14336, fmt="bfp4", what="Llama-3-8B MLP gate/up: two [14336,4096] bfloat4_b, f32 column scales, SwiGLU"),
    "c3": dict(k=14336, n=4096, fmt="bfp8", what="Llama-3-8B MLP down: [4096,14336] bfloat8_b + f32 residual, f32 out"),
    "c5": dict(k=4096, n=151936, fmt="bfp8", what="LM head [151936,4096] bfloat8_b, top-8 records per 2048 columns"),
    # the sibling streamer (int4/w4a16.py of the reference): the gate and up weights of config 2 as one int4 weight
    "w4": dict(k=4096, n=28672, fmt="int4", what="int4 codes with bf16 group scales (G = 32): [28672,4096], one token"),
    # ... and ternary_matmul/t2.py: the same shape in trits with G = 128, the block Hadamard in front (inside the kernel)
    "t2": dict(k=4096, n=28672, fmt="int4", what="ternary weight (G = 128) behind the block Hadamard: [28672,4096], one token"),
    # ... and moe/moe8.py: one token through a layer's chosen experts (the two launches gate_up and down)
    "moe": dict(k=2048, n=768, fmt="bfp4", experts=128, chosen=8,
                what="MoE layer, one token: 8 of 128 bfloat4_b experts [2048 -> 2 x 768 -> 2048] (the expert shape of "
                     "Qwen3-30B-A3B, synthetic weights), gate_up (SwiGLU, routing weights) then down"),
}
BYTES_PER_WEIGHT = {"bfp8": 1.0625, "bfp4": 0.5625, "bf16": 2.0, "int4": 0.5625}
L2_BYTES = 126 * 1024 * 1024


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text())["hbm_gbs"], "measured (MEASURED_PEAKS.json: torch copy, read+write)"
    return 6650.0, "fallback (earlier measurement on this pool)"


class Clocks:
    """nvidia-smi sampled every 200 ms while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        good = [r for r in self.rows if len(r) == 7 and r[0].isdigit()]
        if not good:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in good)]
        return {"sm_mhz": statistics.median(int(r[0]) for r in good), "sm_max_mhz": int(good[0][1]),
                "samples": len(good), "reasons": reasons}


def make_inputs(wl, m, seed, n=None):
    """Seeded synthetic tensors of the workload's shapes: W ~ N(0,1) * 0.02, x ~ N(0,1), scales ~ U(0.5,1.5)."""
    g = torch.Generator().manual_seed(seed)
    k, n = wl["k"], n or wl["n"]
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    return g, x, k, n


def build_gpu_case(name, m, device, copies, seed0, n_cols=None):
    """The device-side tensors of one workload (n_cols: this rank's columns of it, when it is split): `copies` distinct
    packed weight sets, and a closure running step i."""
    from common import ttnn_like as ttnn
    from dense_reader import linear

    wl = WORKLOADS[name]
    dt = {"bfp8": ttnn.bfloat8_b, "bfp4": ttnn.bfloat4_b, "int4": None}[wl["fmt"]]
    g, x, k, n = make_inputs(wl, m, seed0, n_cols)
    tx = ttnn.from_torch(x.reshape(1, 1, m, k), dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT, device=device)
    sets = []
    for c in range(copies):
        gw = torch.Generator().manual_seed(seed0 + 1 + c)
        if name == "t2":
            from ternary_matmul import t2

            u = torch.randint(0, 2000, (n, k), generator=gw, dtype=torch.int16)
            trits = torch.where(u < 600, 0, torch.where(u % 2 == 0, 1, -1)).to(torch.int8)
            scales = (0.01 + 0.02 * torch.rand(n, k // 128, generator=gw)).to(torch.float16)
            sets.append((t2.packed(t2.ternary_weight(device, trits, fmt="bfp4"),
                                   t2.group_scales(device, scales, t2.HADAMARD_SCALE), 128),))
        elif name == "w4":
            from int4 import w4a16

            codes = torch.randint(-7, 8, (n, k), generator=gw).to(torch.int8)
            scales = (torch.rand(n, k // 32, generator=gw) * 0.01 + 0.001).to(torch.bfloat16)
            sets.append((w4a16.packed(w4a16.int4_weight(device, codes), w4a16.group_scales(device, scales)),))
        elif name == "c2":
            wg = linear.native_weight(device, torch.randn(n, k, generator=gw) * 0.02, dt)[0]
            wu = linear.native_weight(device, torch.randn(n, k, generator=gw) * 0.02, dt)[0]
            sets.append((wg, wu))
        else:
            sets.append((linear.native_weight(device, torch.randn(n, k, generator=gw) * 0.02, dt)[0],))
    extra = {}
    if name == "c2":
        sg = (torch.rand(n, generator=g) + 0.5).to(device.torch)
        su = (torch.rand(n, generator=g) + 0.5).to(device.torch)
        y = ttnn.allocate_tensor_on_device([1, 1, m, n], ttnn.bfloat16, ttnn.TILE_LAYOUT, device)

        cs = (sg, su)

        def step(i, x_t=tx, y_t=y, **kw):
            wg, wu = sets[i % copies]
            return linear.matmul(x_t, wg, None, w_up=wu, glu=True, col_scales=cs, out=y_t, **kw)

        def host_step(i, x_pin, y_pin, x_t, y_t, stream, **kw):
            wg, wu = sets[i % copies]
            linear.matmul_host(x_pin, y_pin, x_t, wg, None, w_up=wu, glu=True, col_scales=cs, out=y_t, stream=stream, **kw)
        extra["host_step"] = host_step
        weights = 2
    elif name == "c3":
        res = ttnn.from_torch(torch.randn(1, 1, m, n, generator=g), dtype=ttnn.float32, layout=ttnn.TILE_LAYOUT, device=device)
        y = ttnn.allocate_tensor_on_device([1, 1, m, n], ttnn.float32, ttnn.TILE_LAYOUT, device)

        def step(i, x_t=tx, y_t=y, res_t=res, **kw):
            return linear.matmul(x_t, sets[i % copies][0], None, residual=res_t, out32=True, out=y_t, **kw)

        def host_step(i, x_pin, y_pin, x_t, y_t, stream, **kw):
            linear.matmul_host(x_pin, y_pin, x_t, sets[i % copies][0], None, residual=res, out32=True, out=y_t, stream=stream,
                               **kw)
        extra["host_step"] = host_step
        weights = 1
        extra["res"] = res
    elif name == "c5":
        units = linear.topk_units(n)
        r = linear.topk_result(device, units, 1, 8)
        y = ttnn.allocate_tensor_on_device([1, 1, m, n], ttnn.bfloat16, ttnn.TILE_LAYOUT, device)
        spec = {"r": r, "k": 8, "rows": 1, "slot0": 0, "base": 0, "n": n, "write_y": False}

        top32 = linear.topk_result(device, 1, 1, 32)

        def step(i, x_t=tx, y_t=y, spec_t=spec, merge=True, **kw):
            # the records of every 2048-column unit, then the best 32 of them all (with an exchange: of all ranks')
            linear.matmul(x_t, sets[i % copies][0], None, topk=spec_t, out=y_t, **kw)
            return linear.topk_merge(spec_t["r"], 1, 8, 32, out=top32) if merge else spec_t["r"]
        weights = 1
        extra.update(launches=2, spec=spec, top32=top32)
    elif name == "t2":
        from ternary_matmul import t2

        mask = t2.hadamard_signs(device, torch.where(torch.rand(k, generator=g) < 0.5, -1.0, 1.0))
        y = ttnn.allocate_tensor_on_device([1, 1, m, n], ttnn.bfloat16, ttnn.TILE_LAYOUT, device)

        def step(i, x_t=tx, y_t=y, **kw):
            # one launch: the stream kernel rotates its own copy of x first
            return linear.matmul(x_t, sets[i % copies][0], None, out=y_t, hadamard=mask, **kw)

        def host_step(i, x_pin, y_pin, x_t, y_t, stream, **kw):
            linear.matmul_host(x_pin, y_pin, x_t, sets[i % copies][0], None, out=y_t, stream=stream, hadamard=mask, **kw)
        extra["host_step"] = host_step
        weights = 1
    else:
        y = ttnn.allocate_tensor_on_device([1, 1, m, n], ttnn.bfloat16, ttnn.TILE_LAYOUT, device)

        def step(i, x_t=tx, y_t=y, **kw):
            return linear.matmul(x_t, sets[i % copies][0], None, out=y_t, **kw)

        def host_step(i, x_pin, y_pin, x_t, y_t, stream, **kw):
            linear.matmul_host(x_pin, y_pin, x_t, sets[i % copies][0], None, out=y_t, stream=stream, **kw)
        extra["host_step"] = host_step
        weights = 1
    wbytes = int(weights * k * n * BYTES_PER_WEIGHT[wl["fmt"]])
    # algorithmic bytes of one launch: the weight stream once, x, scales, residual, output
    other = m * k * 2
    other += {"c2": 2 * n * 4 + m * n * 2, "c3": 2 * m * n * 4, "c5": linear.topk_units(n) * 2 * 8 * 4 if name == "c5" else 0,
              "c1": m * n * 2, "w4": m * n * 2, "t2": m * n * 2 + k // 2 * 4}[name]
    return dict(step=step, x=tx, y=y, wbytes=wbytes, abytes=wbytes + other, x_host=x, sets=sets, **extra)


def cpu_reference_arm(name, m, steps, warmup, budget_s=20.0, min_s=3.0):
    """The reference's torch path on the host cores (oracle port): bf16(x).float() @ Wq.float() and the workload's
    output stage, on a column sample, repeated for at least min_s seconds of wall time (and `steps` repetitions, but
    never past budget_s): a few milliseconds of work timed over twenty repetitions moved by 60 % from run to run.
    Returns (GB/s of packed-weight bytes, info)."""
    from oracle import oracle as orc

    wl = WORKLOADS[name]
    torch.set_num_threads(os.cpu_count() or 1)
    k = wl["k"]
    n_s = min(wl["n"], 2048 if name != "c3" else 1024)  # the column sample
    g, x, _, _ = make_inputs(wl, m, 1234)
    gw = torch.Generator().manual_seed(1235)
    nw = 2 if name == "c2" else 1
    if name == "t2":  # (ternary_matmul/t2.py:213-217, :348-350: x rotated, then times q * s in float32)
        u = torch.randint(0, 2000, (n_s, k), generator=gw, dtype=torch.int16)
        trits = torch.where(u < 600, 0, torch.where(u % 2 == 0, 1, -1)).to(torch.int8)
        scales = (0.01 + 0.02 * torch.rand(n_s, k // 128, generator=gw)).to(torch.float16)
        wq = [torch.from_numpy(orc.t2_dequantize(trits.numpy(), scales.to(torch.bfloat16), 128)).T.contiguous()]
        signs = torch.where(torch.rand(k, generator=g) < 0.5, -1.0, 1.0)
        h32 = torch.tensor([[1.0]])
        while h32.shape[0] < 1024:
            h32 = torch.cat([torch.cat([h32, h32], 1), torch.cat([h32, -h32], 1)], 0)
    elif name == "w4":  # (the reference's own host statement: x as bf16 times q * s in float32, int4/w4a16.py:105-107)
        codes = torch.randint(-7, 8, (n_s, k), generator=gw).to(torch.int8)
        scales = (torch.rand(n_s, k // 32, generator=gw) * 0.01 + 0.001).to(torch.bfloat16)
        wq = [torch.from_numpy(orc.int4_dequantized(codes.numpy(), scales)).T.contiguous()]
    else:
        wq = [torch.from_numpy(orc.native_values(torch.randn(n_s, k, generator=gw) * 0.02, wl["fmt"])[0]) for _ in range(nw)]
    sg = torch.rand(n_s, generator=g) + 0.5
    su = torch.rand(n_s, generator=g) + 0.5
    res = torch.randn(m, n_s, generator=g)

    def one():
        if name == "c2":
            gt, up = orc.reference(x, wq[0], sg), orc.reference(x, wq[1], su)
            return (torch.nn.functional.silu(gt) * up).to(torch.bfloat16)
        if name == "c3":
            return orc.reference(x, wq[0]) + res
        if name == "t2":
            xr = ((x.float() * signs).reshape(m, -1, 1024) @ h32.T).reshape(m, k).to(torch.bfloat16)
            return orc.reference(xr, wq[0]).to(torch.bfloat16)
        y = orc.reference(x, wq[0]).to(torch.bfloat16)
        if name == "c5":
            return torch.topk(y.float().reshape(m, -1, min(2048, n_s)), 8, dim=-1)
        return y

    for _ in range(max(3, warmup)):
        one()
    t0 = time.perf_counter()
    done = 0
    while True:
        one()
        done += 1
        el = time.perf_counter() - t0
        if el >= budget_s or (el >= min_s and done >= steps):
            break
    dt = (time.perf_counter() - t0) / done
    sample_bytes = nw * k * n_s * BYTES_PER_WEIGHT[wl["fmt"]]
    info = {"cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n_s} of {wl['n']} columns per weight, {done} steps, fp32 dequantised weights resident in host memory",
            "ms_per_step_sample": dt * 1e3}
    return sample_bytes / dt / 1e9, info


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=600)
    ap.add_argument("--warmup", type=int, default=30)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--ks", type=int, default=0, help="k per slice of the kernel's work items (0: the library's default)")
    ap.add_argument("--cols", type=int, default=0, help="output columns instead of the workload's own (for experiments)")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak",
                    help="N > 1: weak: every rank streams a whole workload; strong: the one workload's columns are split")
    ap.add_argument("--exchange", choices=["fused", "nccl", "none"], default="fused",
                    help="N > 1: how every rank gets all ranks' outputs (fused: peer stores from the stream kernel)")
    ap.add_argument("--lanes", type=int, default=4,
                    help="calls in flight in the end-to-end leg at N = 1 (streams taking the steps in turn; N > 1: two)")
    ap.add_argument("--profile", action="store_true",
                    help="for a profiler: warm-up, then `steps` plain launches (no graph, no e2e, no CPU leg, no JSON line)")
    args = ap.parse_args()
    # stdout carries the one JSON line and nothing else: whatever libraries print there (NCCL's version banner) goes to
    # stderr; emit() puts the line on the real stdout
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(line):
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(line) + "\n").encode())

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    wl = dict(WORKLOADS[args.workload])
    if args.cols:
        wl["n"] = args.cols
    m = args.rows
    steps, warmup = args.steps, max(3, args.warmup)
    config = {"workload": f"{args.workload}: {wl['what']}", "rows": m, "K": wl["k"], "N": wl["n"], "format": wl["fmt"],
              "arithmetic": "bf16 activations x block-float weights (exact products), fp32 accumulation"}
    if wl["fmt"] == "int4":
        config["arithmetic"] = "bf16 activations x int4 codes (exact products), fp32 sums per 32 k, times the bf16 group scale in fp32"

    if args.workload == "moe":
        config.update(K=None, N=None, hidden=wl["k"], intermediate=wl["n"], experts=wl["experts"], chosen=wl["chosen"])
        return moe_main(args, emit, config, steps, warmup)
    if args.impl == "reference":
        if rank != 0:
            return 0
        val, info = cpu_reference_arm(args.workload, m, steps, warmup, budget_s=60.0, min_s=5.0)
        line = {
            "impl": "reference", "metric": "weight_stream_gbps", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warmup, "ms_per_step": info["ms_per_step_sample"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
            "cpu_baseline": {"value": val, "unit": "GB/s", **info},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference's torch CPU path (dense_reader/linear.py:166-169) as restated by the oracle; its device"
                    " path (ttnn on a Tensix simulator) cannot run here",
        }
        emit(line)
        return 0

    from common import ttnn_like as ttnn
    from dense_reader import linear

    if args.ks:
        linear.KS = args.ks
    fused = args.exchange == "fused"
    if world > 1 and not fused:
        # NCCL's all-gather kernel needs SMs of its own to run beside the persistent stream kernel (one CTA per SM; its
        # CTAs fill an SM's shared memory, so NCCL's cannot share one with them), and few channels: it moves a few KB
        linear.MAX_CTAS = torch.cuda.get_device_properties(local).multi_processor_count - 8
        os.environ.setdefault("NCCL_MAX_NCHANNELS", "4")
        os.environ.setdefault("NCCL_MIN_NCHANNELS", "1")
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    device = ttnn.open_device(local)
    # the columns of this rank: weak scaling: a whole workload each (a layer N times as wide); strong: its share of the one
    n_loc, col_start, n_total = wl["n"], rank * wl["n"], world * wl["n"]
    if args.scaling == "strong" and world > 1:
        from dense_reader import sharded

        shards = sharded.column_shards(wl["n"], world, unit=2048 if args.workload == "c5" else 128)
        (col_start, col_end), n_total = shards[rank], wl["n"]
        n_loc = col_end - col_start
    # (the same count on every rank, from the largest shard: every rank must make the same number of exchanged calls)
    n_max = n_loc if not (args.scaling == "strong" and world > 1) else max(b - a for a, b in shards)
    copies = max(2, -(-2 * L2_BYTES // int((2 if args.workload == "c2" else 1) * wl["k"] * n_max * BYTES_PER_WEIGHT[wl["fmt"]])) + (2 if args.scaling == "strong" and world > 1 else 1))
    copies = min(copies, 40)
    if world > 1:
        assert args.scaling == "weak" or fused, "bench: --scaling strong goes with the fused exchange"
        config["columns_per_rank"] = n_loc
    case = build_gpu_case(args.workload, m, device, copies, seed0=100 + 1000 * rank, n_cols=n_loc)
    step = case["step"]
    launches_per_step = case.get("launches", 1)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def join_side():
        pass

    # ---- N > 1: every rank ends each step with all ranks' outputs (or top-k records). "fused": the stream kernel
    # stores them into the other ranks' buffers itself and ends when every rank's have arrived (no collective launch);
    # "nccl": an all-gather per step, on a side stream so that it overlaps the next step's kernel. ----
    exchange_note = "none (one GPU)"
    if world > 1 and fused:
        from dense_reader import sharded

        plain_step = step
        # The LM head's step merges all ranks' records itself, so its kernel must end with every rank's part here. The
        # other workloads' outputs are consumed by whatever comes after the step: the kernel only stores, the call is
        # announced from a second stream, and the wait sits where the bench consumes (the end of the timed region).
        deferred = args.workload != "c5"
        ex = sharded.Exchange(device, 64 << 20, wait="deferred" if deferred else True)
        nbuf = 2
        exchange_note = ("in the stream kernel: peer stores of every output element / record into all ranks' buffers over"
                         " NVLink; " + ("each call announced by a one-thread kernel on a second stream (its fence and the"
                                        " flags' flight overlap the next call), all calls waited for at the end of the timed region"
                                        if deferred else "completion flags, the kernel ends when every rank's part has arrived"))
        def join_side():  # noqa: F811  (the last step's exchange)
            ex.wait_all(linear.status_word(device))

        if args.workload == "c5":
            r0 = case["spec"]["r"]
            strong = args.scaling == "strong"
            units_all = linear.topk_units(n_total) if strong else world * linear.topk_units(n_loc)
            slot0 = col_start // 2048 if strong else rank * linear.topk_units(n_loc)
            recs = [ex.tensor([1, 1, units_all, r0.shape[-1]], r0.dtype) for _ in range(nbuf)]
            case["exchanged_records"] = recs
            specs = [{"r": r, "k": 8, "rows": 1, "slot0": slot0, "base": col_start, "n": n_loc, "write_y": False}
                     for r in recs]

            def step(i):
                return plain_step(i, spec_t=specs[i % nbuf], exchange=ex)
        else:
            outs = [ex.tensor([1, 1, m, n_total], case["y"].dtype) for _ in range(nbuf)]
            kw = {}
            if args.workload == "c3":  # the residual in the gathered output's coordinates
                g = torch.Generator().manual_seed(77)
                kw["res_t"] = ttnn.from_torch(torch.randn(1, 1, m, n_total, generator=g), dtype=ttnn.float32,
                                              layout=ttnn.TILE_LAYOUT, device=device)
                case["res_gathered"] = kw["res_t"]

            def step(i):
                return plain_step(i, y_t=outs[i % nbuf], col0=col_start // 32, exchange=ex, **kw)
    elif world > 1 and args.exchange == "none":
        exchange_note = "none: every rank keeps its own columns (a diagnostic, not the path's result)"
    elif world > 1 and args.workload != "c5":
        exchange_note = "NCCL all-gather of every rank's output per step on a side stream, inside the timed region"
        ybuf = [case["y"], ttnn.allocate_tensor_on_device(case["y"].shape, case["y"].dtype, ttnn.TILE_LAYOUT, device)]
        gbuf = [torch.empty(world * ybuf[0].t.numel(), dtype=ybuf[0].t.dtype, device=device.torch) for _ in range(2)]
        side = torch.cuda.Stream()
        plain_step = step

        def step(i):
            main = torch.cuda.current_stream()
            if i >= 2:
                main.wait_stream(side)  # the gather that read this output buffer two steps ago
            plain_step(i, y_t=ybuf[i % 2])
            side.wait_stream(main)
            with torch.cuda.stream(side):
                dist.all_gather_into_tensor(gbuf[i % 2], ybuf[i % 2].t.reshape(-1))
            return ybuf[i % 2]

        def join_side():  # noqa: F811
            torch.cuda.current_stream().wait_stream(side)
    elif world > 1:
        exchange_note = "NCCL all-gather of every rank's top-k records per step, inside the timed region"
        r0 = case["spec"]["r"]
        rbuf = ttnn.from_torch(torch.zeros(1, 1, world * r0.shape[-2], r0.shape[-1], dtype=torch.int32), dtype=ttnn.uint32,
                               layout=ttnn.ROW_MAJOR_LAYOUT, device=device)
        plain_step5 = step

        def step(i):  # noqa: F811
            r = plain_step5(i, merge=False)
            dist.all_gather_into_tensor(rbuf.t.reshape(-1), r.t.reshape(-1))
            return linear.topk_merge(rbuf, 1, 8, 32, out=case["top32"])

    # ---- N > 1: the exchanged buffer against an NCCL all-gather of the ranks' own results, bit for bit ----
    exchange_check = None
    if world > 1 and fused:
        exchange_check = check_exchange(args.workload, case, step, join_side, device, world, rank, m, n_loc, col_start,
                                        n_total, args.scaling == "strong", shards if args.scaling == "strong" else None)
        if not exchange_check["ok"]:
            sys.stderr.write(f"bench: rank {rank}: the exchanged buffer differs from the gathered results: {exchange_check}\n")
            os._exit(3)

    # ---- device-resident: the K steps as one CUDA graph ----
    if args.profile:
        for i in range(warmup + steps):
            step(i)
        join_side()
        linear.check_status(device)
        return 0
    with Clocks(local) as clk:
        ms, reps, graphed = timed_graph(step, join_side, steps, warmup, world, device, min_s=0.6)
    linear.check_status(device)
    wb = torch.tensor([case["wbytes"]], dtype=torch.float64, device=device.torch)
    if world > 1:
        dist.all_reduce(wb)  # all ranks' packed-weight bytes of one step
    job_bytes = float(wb.item())
    value = job_bytes * steps / (ms * 1e-3) / 1e9
    us_call = ms * 1e3 / steps

    # ---- end to end through the public API with host buffers ----
    e2e = None
    if case.get("host_step") is not None and not (world > 1 and (args.workload == "c3" or not fused)):
        e2e = end_to_end(args.workload, case, wl, m, device, world, rank, n_total, col_start, copies, min(steps, 300),
                         warmup, job_bytes, fused, args.lanes if world == 1 else min(args.lanes, 2))
    linear.check_status(device)

    # ---- what else the metric names, timed in the same run ----
    subs = {}
    if world == 1 and args.workload == "c2" and m == 1 and not args.cols:
        for key, rows in (("sub", 1), ("rows32", 32)):
            subs[key] = sub_case("c3", rows, device, max(50, steps // 3))
        subs["int4"] = sub_case("w4", 1, device, max(50, steps // 3))
        subs["ternary"] = sub_case("t2", 1, device, max(50, steps // 3))
        subs["moe"] = moe_sub_case(device, max(48, steps // 4))
    if args.workload == "c2" and m == 1 and not args.cols and (world == 1 or fused):
        subs["c5_strong"] = lm_head_strong(device, world, rank, max(30, steps // 10))
    linear.check_status(device)

    if rank != 0:
        finish(world)
        return 0
    peak, peak_src = peaks()
    achieved = case["abytes"] / (us_call * 1e-6) / 1e9
    line = {
        "metric": "weight_stream_gbps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms / steps, "us_per_call": us_call, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {**config, "l2": f"rotation over {copies} distinct packed weight sets ({copies * case['wbytes'] / 1e6:.0f} MB > 2 x L2)",
                   "timing": (f"CUDA graph of {steps} launches, {reps} replays, CUDA events" if graphed
                              else f"{steps} plain launches x {reps}, CUDA events"),
                   "exchange": exchange_note},
        "pct_of_8000": 100 * value / world / 8000.0,
        "clocks": clk.summary(),
        "gpu_launches": steps * reps * launches_per_step,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": TRAFFIC.get(args.workload) if m == 1 else None, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": case["abytes"]},
    }
    if e2e is not None:
        line["e2e"] = e2e
    if exchange_check is not None:
        line["exchange_check"] = exchange_check
    line.update(subs)
    if world == 1 and not args.no_cpu:
        val, info = cpu_reference_arm(args.workload, m, 50, 3, budget_s=15.0, min_s=4.0)
        line["cpu_baseline"] = {"value": val, "unit": "GB/s", **info}
    emit(line)
    finish(world)
    return 0


def _barrier(world):
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        torch.cuda.synchronize()


def _max_over_ranks(v, world, device):
    t = torch.tensor([v], device=device.torch)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed_graph(step, join, steps, warmup, world, device, min_s=0.3):
    """`warmup` calls, then `steps` calls captured in one CUDA graph and replayed for at least min_s seconds between
    two CUDA events (after a barrier; the maximum over ranks). Returns (ms per replay, replays, whether a graph was used)."""
    from dense_reader import linear

    for i in range(warmup):
        step(i)
    join()
    linear.check_status(device)
    graph = torch.cuda.CUDAGraph()
    cap = torch.cuda.Stream()
    cap.wait_stream(torch.cuda.current_stream())
    graphed = True
    try:
        with torch.cuda.stream(cap):
            step(0)
            join()
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=cap):
                for i in range(steps):
                    step(i)
                join()
        torch.cuda.synchronize()
        graph.replay()  # one untimed replay
    except Exception as e:  # (a collective that cannot be captured: time plain launches instead)
        graphed = False
        sys.stderr.write(f"bench: CUDA graph capture failed ({type(e).__name__}: {e}); timing plain launches\n")
        torch.cuda.synchronize()

    def run_once():
        if graphed:
            graph.replay()
        else:
            for i in range(steps):
                step(i)
            join()

    _barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    time.sleep(0.25)
    reps = max(1, int(min_s / max(1e-6, steps * 12e-6)))  # keep the timed region long enough for a clock sample
    e0.record()
    for _ in range(reps):
        run_once()
    e1.record()
    torch.cuda.synchronize()
    time.sleep(0.15)
    return _max_over_ranks(e0.elapsed_time(e1) / reps, world, device), reps, graphed


def check_exchange(name, case, step, join, device, world, rank, m, n_loc, col_start, n_total, strong, shards):
    """Every rank runs one step with the in-kernel exchange and one without, the plain results are all-gathered with
    NCCL, and the exchange buffer must hold exactly that: evidence that the peer stores over NVLink land where they
    should, in every rank's buffer."""
    import torch.distributed as dist

    from dense_reader import linear, sharded

    out = step(0)  # exchanged: this rank's part into every rank's buffer
    join()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    if name == "c5":
        # the records of this rank's columns, made without an exchange, with the exchanged call's numbering
        units_loc = linear.topk_units(n_loc)
        umax = torch.tensor([units_loc], device=device.torch)
        dist.all_reduce(umax, op=dist.ReduceOp.MAX)
        umax = int(umax.item())
        r = linear.topk_result(device, umax, 1, 8)
        spec = {"r": r, "k": 8, "rows": 1, "slot0": 0, "base": col_start, "n": n_loc, "write_y": False}
        case["step"](0, spec_t=spec, merge=False)
        torch.cuda.synchronize()
        gathered = sharded.gather_records(r.t.reshape(umax, -1))
        counts = [torch.zeros(1, dtype=torch.int64, device=device.torch) for _ in range(world)]
        dist.all_gather(counts, torch.tensor([units_loc], dtype=torch.int64, device=device.torch))
        want = torch.cat([gathered[q * umax : q * umax + int(c.item())] for q, c in enumerate(counts)])
        got = case["exchanged_records"][0].t.reshape(-1, want.shape[-1])[: want.shape[0]]
    else:
        kw = {}
        if "res_gathered" in case:  # the plain call adds this rank's columns of the same residual
            from common import ttnn_like as ttnn

            part = case["res_gathered"].t[..., col_start : col_start + n_loc].contiguous()
            kw["res_t"] = ttnn.Tensor(part, case["res_gathered"].dtype, ttnn.TILE_LAYOUT, device, None)
        case["step"](0, **kw)  # plain: this rank's columns only, into its own output
        torch.cuda.synchronize()
        widths = [b - a for a, b in shards] if strong else [n_loc] * world
        starts = [a for a, _ in shards] if strong else [q * n_loc for q in range(world)]
        want = sharded.gather_outputs(case["y"].t.reshape(m, -1), [(s0, s0 + w) for s0, w in zip(starts, widths)])
        got = out.t.reshape(m, -1)
    ok = bool(torch.equal(got.reshape(-1).view(torch.uint8), want.contiguous().reshape(-1).view(torch.uint8)))
    t = torch.tensor([int(ok)], device=device.torch)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return {"ok": bool(t.item()), "ranks": world, "compared_bytes": int(want.numel() * want.element_size()),
            "against": "NCCL all-gather of every rank's own result, bit for bit, on every rank"}


def end_to_end(name, case, wl, m, device, world, rank, n_total, col_start, copies, e_steps, warmup, job_bytes, fused, nlanes=2):
    """The same metric with the activations and the result in pinned host memory: every step is one library call
    (tkd_matmul_host: the copy of x to the device, the launch, the copy of the result back), nlanes lanes (stream, staging
    tensors, pinned buffers, workspace; with N > 1 an exchange of its own) taking the steps in turn so that one step's
    copies overlap another's kernel. The calls are independent of each other, so a call's last CTAs (the work split leaves
    some SMs idle at the end of a launch) run beside the next call's first: with four lanes a step takes less than a
    launch does in the device-resident figure, where every launch is ordered behind the one before (measured on config 2:
    21.2 us with two lanes, 18.2 with three, 17.1 with four, 17.9 with six, 20.1 with eight; the launch alone 18.5). Beside
    it the latency of one call at a time (the call, then a synchronise)."""
    from common import ttnn_like as ttnn
    from dense_reader import linear, sharded

    host_call = case["host_step"]
    out_shape = [1, 1, m, n_total if world > 1 else case["y"].shape[-1]]
    x_pin = case["x_host"].reshape(1, 1, m, wl["k"]).contiguous().pin_memory()
    lanes = []
    for ln in range(nlanes):
        ex = sharded.Exchange(device, 4 << 20) if world > 1 and fused else None
        y = (ex.tensor(out_shape, case["y"].dtype) if ex is not None
             else ttnn.allocate_tensor_on_device(out_shape, case["y"].dtype, ttnn.TILE_LAYOUT, device))
        lanes.append(dict(
            stream=torch.cuda.Stream(), slot=1 + ln, ex=ex, y=y,
            x=ttnn.from_torch(torch.zeros(1, 1, m, wl["k"], dtype=torch.bfloat16), dtype=ttnn.bfloat16,
                              layout=ttnn.TILE_LAYOUT, device=device),
            xp=x_pin.clone().pin_memory(), yp=torch.empty(out_shape, dtype=y.t.dtype).pin_memory()))

    def call(i, ln):
        linear.WORKSPACE_SLOT = ln["slot"]
        kw = {} if ln["ex"] is None else {"exchange": ln["ex"], "col0": col_start // 32}
        host_call(i, ln["xp"], ln["yp"], ln["x"], ln["y"], ln["stream"], **kw)
        linear.WORKSPACE_SLOT = 0

    def join():
        for ln in lanes:
            if ln["ex"] is not None:
                ln["ex"].wait_all(linear.status_word(device), stream=ln["stream"])
            torch.cuda.current_stream().wait_stream(ln["stream"])

    def fork():
        for ln in lanes:
            ln["stream"].wait_stream(torch.cuda.current_stream())

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fork()
    for i in range(max(warmup, 2 * copies)):
        call(i, lanes[i % nlanes])
    join()

    def timed(n):
        _barrier(world)
        fork()
        e0.record()
        for i in range(n):
            call(i, lanes[i % nlanes])
        join()
        e1.record()
        torch.cuda.synchronize()
        return _max_over_ranks(e0.elapsed_time(e1), world, device)

    # the e_steps calls once, then as many times over as fill a quarter of a second (a few hundred microseconds of calls
    # paced by the host moved by 10 % from run to run); the figure is per call of the longer run
    e2e_ms, reps = timed(e_steps), 1
    want = int(250.0 / max(e2e_ms, 1e-3))
    if want > 1:
        reps = max(1, min(want, 20000 // max(e_steps, 1)))
        e2e_ms = timed(e_steps * reps) / reps
    linear.check_status(device)
    # one call at a time: host wall clock around call + synchronise (a decode step that needs its result before the next)
    lat_steps = min(e_steps, 100)
    _barrier(world)
    t0 = time.perf_counter()
    for i in range(lat_steps):
        call(i, lanes[0])
        lanes[0]["stream"].synchronize()
    lat_us = _max_over_ranks((time.perf_counter() - t0) / lat_steps * 1e6, world, device)
    linear.check_status(device)
    return {"value": job_bytes * e_steps / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "us_per_call": e2e_ms * 1e3 / e_steps,
            "steps": e_steps, "reps": reps, "mode": f"pipelined x{nlanes} ({nlanes} calls in flight on {nlanes} streams)",
            "h2d_bytes_per_step": x_pin.numel() * 2, "d2h_bytes_per_step": lanes[0]["yp"].numel() * lanes[0]["yp"].element_size(),
            "one_call_at_a_time_us": lat_us}



# ---- the mixture-of-experts sibling (moe/moe8.py of the reference): a workload of its own, two launches a step ----


def moe_layer_bytes(wl, experts):
    """Packed-weight bytes of `experts` experts of the layer: gate|up [H, 2I] and down [I, H] at 0.5625 bytes a weight."""
    return int(experts * 3 * wl["k"] * wl["n"] * BYTES_PER_WEIGHT["bfp4"])


def build_moe_case(device, rows, seed0):
    """The packed layer (made on the GPU from seeded normal weights), one activation row (or `rows` of them with their own
    experts), and id sets that together go through all experts, so that a step's experts are never in L2 (all experts:
    340 MB): step i runs gate_up then down on set i."""
    from common import ttnn_like as ttnn
    from moe import moe8

    wl = WORKLOADS["moe"]
    E, H, I, K = wl["experts"], wl["k"], wl["n"], wl["chosen"]
    g = torch.Generator(device=device.torch).manual_seed(seed0)
    gu = torch.randn(E, H, 2 * I, generator=g, device=device.torch) * 0.02
    dn = torch.randn(E, I, H, generator=g, device=device.torch) * 0.02
    P = moe8.pack(device, gu, dn)
    del gu, dn
    gc = torch.Generator().manual_seed(seed0 + 1)
    x = torch.randn(rows, H, generator=gc).to(torch.bfloat16)
    tx = ttnn.from_torch(x.reshape(1, 1, rows, H), dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT, device=device)
    sets, experts_read = [], []
    perm = torch.randperm(E, generator=gc)
    for s in range(E // K if rows == 1 else 8):
        if rows == 1:
            ids = perm[s * K:(s + 1) * K].reshape(1, K)
        else:
            ids = torch.stack([torch.randperm(E, generator=gc)[:K] for _ in range(rows)])
        w = torch.softmax(torch.randn(rows, K, generator=gc), -1).to(torch.bfloat16)
        sets.append((ttnn.from_torch(ids.to(torch.int16).reshape(1, 1, rows, K), dtype=ttnn.uint16, layout=ttnn.TILE_LAYOUT, device=device),
                     ttnn.from_torch(w.reshape(1, 1, rows, K), dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT, device=device)))
        experts_read.append(len(moe8.union(ids, E)))

    def step(i, x_t=tx):
        tid, tw = sets[i % len(sets)]
        if rows == 1:
            return moe8.down(moe8.gate_up(x_t, P, tid, tw, K), P, tid, K)
        return moe8.down_rows(moe8.gate_up_rows(x_t, P, tid, tw, K, rows), P, tid, K, rows)

    nread = sum(experts_read) / len(experts_read)
    wbytes = moe_layer_bytes(wl, nread)
    # algorithmic bytes of a step: the chosen experts' weights once, x, ids and routing weights, h written and read, y
    um = K if rows == 1 else min(E, rows * K)
    other = rows * H * 2 + rows * K * 4 + 2 * rows * um * I * 2 + rows * H * 2
    return dict(step=step, P=P, x=tx, x_host=x, sets=sets, wbytes=wbytes, abytes=wbytes + other, experts_read=nread)


def moe_cpu_arm(steps, warmup, budget_s, min_s):
    """The reference's own host statement of the layer (moe8.reference, moe/moe8.py:619-636: float64 matmuls over the
    chosen experts' dequantised weights) as the oracle restates it, on a layer of 16 experts resident in host memory."""
    from oracle import oracle as orc

    wl = WORKLOADS["moe"]
    H, I, K, E = wl["k"], wl["n"], wl["chosen"], 16
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(77)
    gu = (torch.randn(E, H, 2 * I, generator=g) * 0.02).to(torch.bfloat16).double().numpy()
    dn = (torch.randn(E, I, H, generator=g) * 0.02).to(torch.bfloat16).double().numpy()
    x = torch.randn(1, H, generator=g).to(torch.bfloat16).double().numpy()
    w = torch.softmax(torch.randn(K, generator=g), 0).double().numpy()
    sets = [torch.randperm(E, generator=g)[:K].tolist() for _ in range(8)]
    for i in range(max(3, warmup)):
        orc.moe_reference(x, gu, dn, sets[i % 8], w)
    t0, done = time.perf_counter(), 0
    while True:
        orc.moe_reference(x, gu, dn, sets[done % 8], w)
        done += 1
        el = time.perf_counter() - t0
        if el >= budget_s or (el >= min_s and done >= steps):
            break
    dt = el / done
    info = {"cores": torch.get_num_threads(), "kind": "port",
            "sample": f"the whole step ({K} experts) on a layer of {E} experts held dequantised in float64, {done} steps",
            "ms_per_step_sample": dt * 1e3}
    return moe_layer_bytes(wl, K) / dt / 1e9, info


def moe_main(args, emit, config, steps, warmup):
    """bench.py --workload moe at N = 1 (more ranks: replicas; the layer has no exchange step of its own here)."""
    from common import ttnn_like as ttnn

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    wl = WORKLOADS["moe"]
    if args.impl == "reference":
        if rank == 0:
            val, info = moe_cpu_arm(steps, warmup, 60.0, 5.0)
            emit({"impl": "reference", "metric": "weight_stream_gbps", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
                  "steps": steps, "warmup": warmup, "ms_per_step": info["ms_per_step_sample"], "higher_is_better": True,
                  "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic", "config": config,
                  "cpu_baseline": {"value": val, "unit": "GB/s", **info},
                  "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        return 0
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    device = ttnn.open_device(local)
    case = build_moe_case(device, args.rows, 100 + 1000 * rank)
    step = case["step"]
    if args.profile:
        for i in range(warmup + steps):
            step(i)
        torch.cuda.synchronize()
        finish(world)
        return 0
    with Clocks(local) as clk:
        ms, reps, graphed = timed_graph(step, lambda: None, steps, warmup, world, device)
    us = ms * 1e3 / steps
    value = world * case["wbytes"] / (us * 1e-6) / 1e9
    # end to end, one call at a time: x from pinned host memory, the two launches, y back
    x_pin = case["x_host"].reshape(1, 1, args.rows, -1).contiguous().pin_memory()
    y_pin = torch.empty(1, 1, 32 if args.rows > 1 else 1, wl["k"], dtype=torch.bfloat16).pin_memory()
    e_steps = min(steps, 200)

    def host_call(i):
        case["x"].t.copy_(x_pin, non_blocking=True)
        y = step(i)
        y_pin.copy_(y.t, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(warmup):
        host_call(i)
    _barrier(world)
    t0 = time.perf_counter()
    for i in range(e_steps):
        host_call(i)
    e_us = _max_over_ranks((time.perf_counter() - t0) / e_steps * 1e6, world, device)
    if rank != 0:
        finish(world)
        return 0
    peak, peak_src = peaks()
    achieved = case["abytes"] / (us * 1e-6) / 1e9
    line = {
        "metric": "weight_stream_gbps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms / steps, "us_per_call": us, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {**config, "experts_read_per_step": case["experts_read"],
                   "l2": f"the steps' id sets go through all {wl['experts']} experts ({moe_layer_bytes(wl, wl['experts']) / 1e6:.0f} MB > 2 x L2)",
                   "timing": (f"CUDA graph of {steps} steps (two launches each), {reps} replays, CUDA events" if graphed
                              else f"{steps} plain steps x {reps}, CUDA events"),
                   "exchange": "none: every rank runs the whole layer (replicas)"},
        "pct_of_8000": 100 * value / world / 8000.0, "clocks": clk.summary(), "gpu_launches": steps * reps * 2,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": TRAFFIC.get("moe") if args.rows == 1 else None, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": case["abytes"],
                     "note": "per step of two launches (gate_up and down); traffic likewise"},
        "e2e": {"value": world * case["wbytes"] / (e_us * 1e-6) / 1e9, "unit": "GB/s", "us_per_call": e_us,
                "mode": "one call at a time", "h2d_bytes_per_step": x_pin.numel() * 2, "d2h_bytes_per_step": y_pin.numel() * 2},
    }
    if world == 1 and not args.no_cpu:
        val, info = moe_cpu_arm(50, 3, 15.0, 4.0)
        line["cpu_baseline"] = {"value": val, "unit": "GB/s", **info}
    emit(line)
    finish(world)
    return 0


def moe_sub_case(device, steps):
    """The MoE layer's record for the default line: one token, then 8 and 32 rows with their own experts."""
    out = {"workload": "moe: " + WORKLOADS["moe"]["what"], "unit": "GB/s"}
    peak, _ = peaks()
    for rows in (1, 8, 32):
        case = build_moe_case(device, rows, 700 + rows)
        n = steps if rows == 1 else max(10, steps // 8)
        ms, _, _ = timed_graph(case["step"], lambda: None, n, 5, 1, device, min_s=0.2)
        us = ms * 1e3 / n
        rec = {"us_per_call": us, "value": case["wbytes"] / (us * 1e-6) / 1e9, "experts_read": case["experts_read"], "launches": 2,
               "roofline": {"bound": "hbm", "achieved": case["abytes"] / (us * 1e-6) / 1e9, "peak": peak, "unit": "GB/s",
                            "frac": case["abytes"] / (us * 1e-6) / 1e9 / peak, "algorithmic_bytes_per_launch": case["abytes"]}}
        if rows == 1:
            out.update(rows=1, **rec)
        else:
            out[f"rows{rows}"] = rec
        del case
        torch.cuda.empty_cache()
    return out


def sub_case(name, rows, device, steps):
    """Another workload at N = 1, device-resident, graph-replayed: microseconds per call and its roofline."""
    wl = WORKLOADS[name]
    copies = min(40, max(2, -(-2 * L2_BYTES // int(wl["k"] * wl["n"] * BYTES_PER_WEIGHT[wl["fmt"]])) + 1))
    case = build_gpu_case(name, rows, device, copies, seed0=500 + rows)
    ms, reps, _ = timed_graph(case["step"], lambda: None, steps, 5, 1, device, min_s=0.2)
    us = ms * 1e3 / steps
    peak, _ = peaks()
    achieved = case["abytes"] / (us * 1e-6) / 1e9
    out = {"workload": f"{name}: {wl['what']}", "rows": rows, "us_per_call": us, "value": case["wbytes"] / (us * 1e-6) / 1e9,
           "unit": "GB/s", "steps": steps,
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                        "algorithmic_bytes_per_launch": case["abytes"]}}
    del case
    torch.cuda.empty_cache()
    return out


def lm_head_strong(device, world, rank, steps):
    """The LM head's 151936 columns split over the ranks by 2048-column units (strong scaling): every rank streams its
    shard, its top-k records go into every rank's buffer from inside the kernel, and every rank merges the global
    top-32. Microseconds per step (max over ranks), with the exchanged records checked against an NCCL gather."""
    from dense_reader import linear, sharded

    wl = WORKLOADS["c5"]
    if world > 1:
        import torch.distributed as dist

        shards = sharded.column_shards(wl["n"], world, unit=2048)
    else:
        shards = [(0, wl["n"])]
    a, b = shards[rank]
    n_loc = b - a
    case = build_gpu_case("c5", 1, device, 2 if world > 1 else 1, seed0=900 + rank, n_cols=n_loc)
    step, join, check = case["step"], (lambda: None), None
    if world > 1:
        ex = sharded.Exchange(device, 1 << 20)
        r0 = case["spec"]["r"]
        units_all = linear.topk_units(wl["n"])
        recs = [ex.tensor([1, 1, units_all, r0.shape[-1]], r0.dtype) for _ in range(2)]
        specs = [{"r": r, "k": 8, "rows": 1, "slot0": a // 2048, "base": a, "n": n_loc, "write_y": False} for r in recs]
        plain = case["step"]
        case["exchanged_records"] = recs

        def step(i):  # noqa: F811
            return plain(i, spec_t=specs[i % 2], exchange=ex)

        def join():  # noqa: F811
            ex.wait_all(linear.status_word(device))

        check = check_exchange("c5", case, step, join, device, world, rank, 1, n_loc, a, wl["n"], True, shards)
    ms, reps, _ = timed_graph(step, join, steps, 5, world, device, min_s=0.2)
    linear.check_status(device)
    out = {"workload": f"c5: {wl['what']}", "us_per_call": ms * 1e3 / steps, "columns_per_rank": n_loc, "steps": steps,
           "value": wl["k"] * wl["n"] * BYTES_PER_WEIGHT[wl["fmt"]] / (ms * 1e-3 / steps) / 1e9, "unit": "GB/s",
           "launches_per_step": 2}
    if check is not None:
        out["exchange_check"] = check
    del case
    torch.cuda.empty_cache()
    return out


def finish(world):
    """Leave a multi-rank run without waiting on NCCL's teardown (captured collectives can keep it from returning)."""
    if world > 1:
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


# DRAM bytes per launch of tkd_stream_kernel from an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum), per
# workload at M = 1 (the summaries under profiles/); None where no capture of the workload is summarised there.
TRAFFIC = {"c2": 66_769_408, "c3": 62_681_600, "c5": 667_036_928, "w4": 66_386_432, "moe": 21_298_944}

if __name__ == "__main__":
    sys.exit(main())
