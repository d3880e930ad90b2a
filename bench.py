#!/usr/bin/env python
"""Benchmark of the block-sparse attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME]

Workload (default `stride_bertbase`): stride-pattern block-sparse attention at the BERT-base shape,
fp16 storage with fp32 accumulation, B=8 H=12 L=4096 d=64, 64x64 blocks, layout = band of 4 blocks
plus every 8th block column (730 kept blocks per head).  A step is one fused attention launch
(SDDMM + softmax + SpMM in one kernel) over the whole batch.  The metric is TFLOP/s counted on the
kept blocks only: 4 * 64 * 64 * d * blocks * B * H flops per step.

One JSON line is printed by rank 0.  `value` is measured with the operands resident in HBM;
`e2e` goes through the same C-ABI call with the operands in pinned host memory, so the
host->device and device->host copies are inside its timed region.  `--impl reference` times the
reference's own CPU operators (matmul.h / ewops.h, compiled into oracle/_ref) on a bounded sample.
With N > 1 every rank runs the workload on its own batch (batch x head sharding, no collective on
the data path); the NCCL all-gather of the outputs is timed separately as `gather_ms`.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: dtype, B, H, L, d, bs, layout kind + parameters
    "stride_bertbase": dict(dtype="f16", B=8, H=12, L=4096, d=64, bs=64, layout=("LAYOUT_STRIDE", dict(p0=4, p1=8)),
                            oracle=("stride", dict(band=4, every=8))),
    "bigbird": dict(dtype="bf16", B=16, H=12, L=4096, d=64, bs=64,
                    layout=("LAYOUT_BIGBIRD", dict(p0=1, p1=1, p2=1, p3=3, seed=1236)),
                    oracle=("bigbird", dict(window=1, g_first=1, g_last=1, nrand=3, seed=1236))),
    "local_bertlarge": dict(dtype="bf16", B=4, H=16, L=16384, d=64, bs=64, layout=("LAYOUT_LOCAL", dict(p0=8, p1=8)),
                            oracle=("local", dict(left=8, right=8))),
    "full_bertlarge": dict(dtype="bf16", B=32, H=16, L=1024, d=64, bs=64, layout=("LAYOUT_FULL", dict()),
                           oracle=("full", dict())),
    "fixed_fp32": dict(dtype="f32", B=1, H=4, L=512, d=64, bs=32, layout=("LAYOUT_FIXED", dict(p0=4)),
                       oracle=("fixed", dict(stride=4)), lut_heads=4),
}


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the fused kernel, from one ncu capture of this
# command line (a profiler cannot run inside the timed region; the line says so in "traffic_source")
NCU_TRAFFIC_BYTES = {"stride_bertbase": 179.7e6}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(tensor=p["bf16_tflops"], tensor_sustained=p["bf16_tflops_sustained"], hbm=p["hbm_gbs"], source="measured")
    return dict(tensor=1590.0, tensor_sustained=1400.0, hbm=6650.0, source="fallback")


class L2Flush:
    """What runs between timed steps: 256 MB written (twice the 126 MB L2) and then, unless mode is "write", 256 MB of a
    second buffer read.  After the write alone the L2 is full of the flush's own dirty lines, and their write-back
    (up to ~120 MB of DRAM writes) would land inside the next timed kernel; after the read it is cold and clean."""

    def __init__(self, torch, mode="write_read"):
        self.mode = mode
        self.w = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        self.r = torch.zeros(64 << 20, dtype=torch.float32, device="cuda") if mode != "write" else None   # summed as it is, no cast pass
        self.note = ("256 MB written then 256 MB read between timed steps (cold and clean)" if mode != "write"
                     else "256 MB written between timed steps")

    def fill_(self, value=1):
        self.w.fill_(value)
        if self.r is not None:
            self.sink = self.r.sum()


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.12)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1])); power.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        # the busy samples are the ones that matter: take the median of the upper half by power
        order = sorted(range(len(sm)), key=lambda i: power[i])
        busy = [sm[i] for i in order[len(order) // 2:]]
        return dict(sm_mhz=statistics.median(busy), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm),
                    power_w_max=max(power))


def attention_flops(cfg, blocks):
    return 4.0 * cfg["bs"] * cfg["bs"] * cfg["d"] * blocks * cfg["B"] * cfg["H"]


def bind_to_gpu_cpus(index):
    """Run this process (and first-touch its pinned buffers) on the CPUs next to its GPU: the end-to-end figure moves
    150 MB per step from host memory, and a buffer on the far socket halves that rate.  Only this process's own CPU
    affinity changes (the caller puts it back before the CPU baseline, which wants every core).  The GPU is looked up
    by its PCI address, which is the same whatever subset of the host's GPUs this process sees.  Returns the number of
    CPUs bound to, or None."""
    try:
        import pynvml
        import torch
        pynvml.nvmlInit()
        pr = torch.cuda.get_device_properties(index)
        try:
            h = pynvml.nvmlDeviceGetHandleByPciBusId("%08x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id))
        except Exception:
            h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None



# ------------------------------------------------------------------------------------------------
def _load_encoder():
    import importlib.util
    spec = importlib.util.spec_from_file_location("sfb_encoder", os.path.join(ROOT, "sf-bert_b200", "encoder.py"))
    enc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(enc)
    return enc


def measure_encoder_layer(torch, sfb, cfg, steps, flush):
    """ms per forward of one post-LN encoder layer at the workload's shape on this rank (attention, projections with
    bias / GELU, bias + residual + LayerNorm all from this library); L2 flushed between timed steps."""
    enc = _load_encoder()
    B, H, L, d, bs = cfg["B"], cfg["H"], cfg["L"], cfg["d"], cfg["bs"]
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16}[cfg["dtype"]]
    hidden, ffn = H * d, 4 * H * d
    lay = sfb.BlockLayout.generate(getattr(sfb, cfg["layout"][0]), cfg.get("lut_heads", 1), L // bs, bs, **cfg["layout"][1])
    w = enc.EncoderLayerWeights(hidden, ffn, tdt, seed=1)
    x = torch.randn(B, L, hidden, device="cuda").to(tdt)
    fn = lambda: enc.encoder_layer(sfb, x, w, lay, H, "post", "tensor")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b_ in ev:
        flush.fill_(1)
        a.record()
        fn()
        b_.record()
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b_) for a, b_ in ev) / steps, B


def measure_encoder_stack(torch, sfb, cfg, steps, layers, rank):
    """ms per forward of embedding + positions + `layers` post-LN encoder layers at the workload's shape, 1/8 of its
    batch on this rank (the workload's 8-GPU split), replayed as one CUDA graph."""
    enc = _load_encoder()
    B, H, L, d, bs = cfg["B"], cfg["H"], cfg["L"], cfg["d"], cfg["bs"]
    Bg = B // 8 if B >= 8 and B % 8 == 0 else B
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16}[cfg["dtype"]]
    hidden, ffn, vocab = H * d, 4 * H * d, 30522
    lay = sfb.BlockLayout.generate(getattr(sfb, cfg["layout"][0]), cfg.get("lut_heads", 1), L // bs, bs, **cfg["layout"][1])
    ws = [enc.EncoderLayerWeights(hidden, ffn, tdt, seed=100 + i) for i in range(layers)]
    g = torch.Generator(device="cuda").manual_seed(7)
    table = (0.02 * torch.randn(vocab, hidden, device="cuda", generator=g)).to(tdt)
    pos = (0.02 * torch.randn(L, hidden, device="cuda", generator=g)).to(tdt)
    ids = torch.randint(0, vocab, (Bg, L), device="cuda", dtype=torch.int32,
                        generator=torch.Generator(device="cuda").manual_seed(1234 + rank))

    def forward(tok):
        x, _ = sfb.embedding(table, tok, pos)
        for w in ws:
            x = enc.encoder_layer(sfb, x, w, lay, H, "post", "tensor")
        return x

    for _ in range(2):
        forward(ids)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        forward(ids)
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        forward(ids)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps, Bg


def pair_slices(B, H, start, stop):
    """The (batch, head) pairs [start, stop) (pair = b * H + h) as rectangles (b0, b1, h0, h1) of the [B, L, H, d] tensors."""
    out = []
    p = start
    while p < stop:
        b, h = divmod(p, H)
        if h == 0 and stop - p >= H:
            nb_ = (stop - p) // H
            out.append((b, b + nb_, 0, H))
            p += nb_ * H
        else:
            h1 = min(H, h + stop - p)
            out.append((b, b + 1, h, h1))
            p += h1 - h
    return out


def measure_strong_scaling(torch, dist, sfb, steps, world, rank, chunks=None):
    """Strong scaling of the `local_bertlarge` workload (B=4, H=16, L=16384: 64 (batch, head) pairs): the pairs are dealt
    contiguously to the ranks (sharding.partition_pairs), a rank computes its share in place on head slices of the full
    tensors (sfb_fused_attention_slice) in `chunks` launches, and every chunk's output is all-gathered (NCCL) on a second
    stream while the next chunk computes.  Returns ms for the share alone, for the gather alone and for both overlapped."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("sfb_sharding", os.path.join(ROOT, "sf-bert_b200", "sharding.py"))
    sh = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sh)
    cfg = CONFIGS["local_bertlarge"]
    B, H, L, d, bs = cfg["B"], cfg["H"], cfg["L"], cfg["d"], cfg["bs"]
    lay = sfb.BlockLayout.generate(getattr(sfb, cfg["layout"][0]), 1, L // bs, bs, **cfg["layout"][1])
    gen = torch.Generator(device="cuda").manual_seed(4321)      # the same tensors on every rank
    q, k, v = (torch.randn(B, L, H, d, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(3))
    start, stop = sh.partition_pairs(B, H, world, rank)
    n = stop - start
    if chunks is None:
        # two chunks (so that a gather can run under the second) only while each still fills the GPU several times over:
        # the kernel deals whole row pairs to 3 streams on each of 148 SMs, and a launch of about as many pairs as streams
        # ends with most of them idle
        row_pairs = (L // bs + 1) // 2
        chunks = 2 if world > 1 and (n // 2) * row_pairs >= 4 * 3 * 148 else 1
    # the share in `chunks` pieces of whole pairs, each piece a few rectangles
    bounds = [start + (n * c) // chunks for c in range(chunks + 1)]
    pieces = [pair_slices(B, H, bounds[c], bounds[c + 1]) for c in range(chunks) if bounds[c + 1] > bounds[c]]
    outs = [[torch.empty(b1 - b0, L, h1 - h0, d, dtype=torch.bfloat16, device="cuda") for (b0, b1, h0, h1) in piece] for piece in pieces]
    gathered = [[torch.empty((world,) + tuple(o.shape), dtype=o.dtype, device="cuda") for o in po] for po in outs] if world > 1 else None
    scale = 1.0 / d ** 0.5
    comm = torch.cuda.Stream()

    def compute(c):
        for (b0, b1, h0, h1), o in zip(pieces[c], outs[c]):
            sfb.fused_attention_slice(q[b0:b1, :, h0:h1], k[b0:b1, :, h0:h1], v[b0:b1, :, h0:h1], lay, scale, out=o)

    def gather(c):
        for o, g_ in zip(outs[c], gathered[c]):
            dist.all_gather_into_tensor(g_, o)

    def run(do_compute, do_gather):
        cur = torch.cuda.current_stream()
        for c in range(len(pieces)):
            if do_compute:
                compute(c)
            if do_gather and world > 1:
                ev = torch.cuda.Event()
                ev.record(cur)
                comm.wait_event(ev)
                with torch.cuda.stream(comm):
                    gather(c)
        if do_gather and world > 1:
            cur.wait_stream(comm)

    def timed(do_compute, do_gather):
        for _ in range(3):
            run(do_compute, do_gather)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            run(do_compute, do_gather)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    ms_share = timed(True, False)
    ms_gather = timed(False, True) if world > 1 else 0.0
    ms_both = timed(True, True) if world > 1 else ms_share
    flops = attention_flops(cfg, lay.blocks)
    return dict(ms_share=ms_share, ms_gather=ms_gather, ms_both=ms_both, flops=flops, pairs=B * H, pairs_here=n,
                launches=sum(len(p_) for p_ in pieces), gather_bytes=sum(o.numel() * 2 for po in outs for o in po))

# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge
    sfb = ge.load_package()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    all_cpus = os.sched_getaffinity(0)
    near = bind_to_gpu_cpus(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = CONFIGS[args.config]
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[cfg["dtype"]]
    B, H, L, d, bs = cfg["B"], cfg["H"], cfg["L"], cfg["d"], cfg["bs"]
    nb = L // bs
    lay = sfb.BlockLayout.generate(getattr(sfb, cfg["layout"][0]), cfg.get("lut_heads", 1), nb, bs, **cfg["layout"][1])
    scale = 1.0 / d ** 0.5

    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    q, k, v = (torch.randn(B, L, H, d, device="cuda", dtype=torch.float32, generator=gen).to(tdt) for _ in range(3))
    o = torch.empty_like(q)
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty_like(hq).pin_memory()
    flush = L2Flush(torch, args.l2_flush)

    def step():
        sfb.fused_attention(q, k, v, lay, scale, out=o)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        flush.fill_(1)
        step()
    sync_all()

    sampler = ClockSampler(local) if rank == 0 else None
    # resident-operand timing: one event pair per step, L2 flushed in between (flush not timed)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    sync_all()
    for a, b_ in ev:
        flush.fill_(1)
        a.record()
        step()
        b_.record()
    sync_all()
    ms_steps = [a.elapsed_time(b_) for a, b_ in ev]
    ms_total = sum(ms_steps)

    # end to end through the same call: pinned host operands in, output back to the host
    # (the package's host pipeline: batch chunks, copies in / kernel / copy out overlapped on three streams)
    pipe = sfb.HostPipeline(tuple(q.shape), tdt, lay, chunks=B)

    def e2e_step():
        pipe(hq, hk, hv, ho, scale)

    for _ in range(3):
        e2e_step()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    sync_all()
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None

    gather_ms = None
    if world > 1:
        outs = torch.empty((world,) + tuple(o.shape), dtype=o.dtype, device="cuda")
        for _ in range(3):
            dist.all_gather_into_tensor(outs, o)
        sync_all()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(5):
            dist.all_gather_into_tensor(outs, o)
        g1.record()
        sync_all()
        gather_ms = g0.elapsed_time(g1) / 5

    # the rest of the metric and of the multi-GPU row, as extra keys of the same line (headline workload only)
    extra = None
    if args.config == "stride_bertbase" and not args.no_extras:
        del hq, hk, hv, ho, pipe
        layer_ms, layer_B = measure_encoder_layer(torch, sfb, cfg, args.steps, flush)
        stack_ms, stack_B = measure_encoder_stack(torch, sfb, CONFIGS["full_bertlarge"], max(args.steps // 2, 3), args.layers, rank)
        strong = measure_strong_scaling(torch, dist, sfb, args.steps, world, rank)
        extra = dict(layer_ms=layer_ms, layer_B=layer_B, stack_ms=stack_ms, stack_B=stack_B, strong=strong)

    status = sfb.device_status()
    vals = [ms_total, e2e_ms, gather_ms or 0.0]
    if extra:
        vals += [extra["layer_ms"], extra["stack_ms"], extra["strong"]["ms_share"], extra["strong"]["ms_gather"], extra["strong"]["ms_both"]]
    t = torch.tensor(vals, dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    vals = [float(x) for x in t.cpu()]
    ms_total, e2e_ms, gather_max = vals[:3]

    if rank == 0:
        pk = peaks()
        flops = attention_flops(cfg, lay.blocks)
        ms_per_step = ms_total / args.steps
        value = world * flops / (ms_per_step * 1e-3) / 1e12
        per_gpu = flops / (ms_per_step * 1e-3) / 1e12
        esz = q.element_size()
        line = {
            "metric": "block-sparse attention TFLOP/s on nonzero blocks",
            "value": round(value, 3), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": cfg["dtype"], "data": "synthetic",
            "config": {"workload": args.config, "B_per_gpu": B, "H": H, "L": L, "d": d, "block": bs,
                       "layout": cfg["layout"][0], "nnz_blocks_per_head": lay.blocks, "max_row": lay.nn_max,
                       "sharding": "batch x head, no collective on the data path", "l2": flush.note},
            "roofline": {"bound": "tensor", "achieved": round(per_gpu, 3), "peak": pk["tensor"], "unit": "TFLOP/s",
                         "frac": round(per_gpu / pk["tensor"], 4), "traffic": NCU_TRAFFIC_BYTES.get(args.config),
                         "traffic_source": "one ncu capture of this command, not this run" if args.config in NCU_TRAFFIC_BYTES else None,
                         "peak_source": pk["source"] + " burst bf16",
                         "frac_of_sustained": round(per_gpu / pk["tensor_sustained"], 4),
                         "min_hbm_bytes": 4 * B * L * H * d * esz,
                         "kernel": "fused_attention_tc_kernel" if cfg["dtype"] != "f32" else "fused_attention_kernel"},
            "e2e": {"value": round(world * flops / (e2e_ms / args.steps * 1e-3) / 1e12, 3), "unit": "TFLOP/s",
                    "ms_per_step": round(e2e_ms / args.steps, 4), "pipeline": "%d batch chunks, 3 streams" % B,
                    "host_cpus_bound": near,
                    "h2d_bytes_per_step": 3 * B * L * H * d * esz, "d2h_bytes_per_step": B * L * H * d * esz},
            "gpu_launches": args.steps * (1 + B),   # resident loop: one fused kernel per step; end-to-end loop: one per batch chunk
            "clocks": clocks, "device_status": status,
        }
        if gather_ms is not None:
            line["gather_ms"] = round(gather_max, 4)
        if extra:
            layer_ms, stack_ms, share_ms, sgather_ms, both_ms = vals[3:8]
            st = extra["strong"]
            line["encoder_layer_seq_s"] = {"value": round(world * extra["layer_B"] / (layer_ms * 1e-3), 1), "unit": "seq/s", "ms_per_layer": round(layer_ms, 4),
                                           "config": "one post-LN encoder layer at the stride_bertbase shape (B=%d per GPU, L=4096, hidden 768, FFN 3072), all kernels from this library" % extra["layer_B"],
                                           "scaling": "weak"}
            line["encoder_stack_seq_s"] = {"value": round(world * extra["stack_B"] / (stack_ms * 1e-3), 1), "unit": "seq/s", "ms_per_forward": round(stack_ms, 4),
                                           "config": "embedding + %d post-LN layers at the full_bertlarge shape (L=1024, hidden 1024, FFN 4096), %d sequences per GPU, one CUDA graph replay per forward" % (args.layers, extra["stack_B"]),
                                           "scaling": "weak"}
            line["strong_scaling"] = {"workload": "local_bertlarge", "pairs": st["pairs"], "pairs_per_rank": st["pairs_here"],
                                      "ms_share": round(share_ms, 4), "gather_ms": round(sgather_ms, 4), "ms_incl_gather": round(both_ms, 4),
                                      "value": round(st["flops"] / (share_ms * 1e-3) / 1e12, 2),
                                      "value_incl_gather": round(st["flops"] / (both_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                                      "how": "the 64 (batch, head) pairs dealt contiguously to the ranks, computed in place on head slices "
                                             "(sfb_fused_attention_slice) in %d launch(es) per step; with two, the first chunk's output is all-gathered on a second stream under the second chunk's compute" % st["launches"],
                                      "gather_bytes_per_rank": st["gather_bytes"], "launches_per_step": st["launches"]}
        if world == 1 and not args.no_cpu:
            os.sched_setaffinity(0, all_cpus)      # the reference's CPU path is timed on every core
            line["cpu_baseline"] = cpu_reference_sample(cfg, budget_s=20.0, steps=1)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
def run_encoder_stack(args):
    """Sequences per second of the whole encoder forward at the workload's shape: embedding lookup + positions, then
    `--layers` post-LN encoder layers (attention, projections, LayerNorm, GELU all from this library), one process per
    GPU with its own slice of the batch (weights replicated, nothing exchanged inside the stack), and an all-gather
    of the outputs afterwards, timed separately.  Weak scaling: the batch per GPU is the workload's batch divided by 8
    (its 8-GPU split) when it is at least 8, else the whole batch."""
    import importlib.util
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge
    sfb = ge.load_package()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    spec = importlib.util.spec_from_file_location("sfb_encoder", os.path.join(ROOT, "sf-bert_b200", "encoder.py"))
    enc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(enc)
    cfg = CONFIGS[args.config]
    B, H, L, d, bs = cfg["B"], cfg["H"], cfg["L"], cfg["d"], cfg["bs"]
    Bg = B // 8 if B >= 8 and B % 8 == 0 else B
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[cfg["dtype"]]
    hidden, ffn, vocab = H * d, 4 * H * d, 30522
    proj = "tensor" if args.projections == "tensor" and tdt != torch.float32 else "library"
    lay = sfb.BlockLayout.generate(getattr(sfb, cfg["layout"][0]), cfg.get("lut_heads", 1), L // bs, bs, **cfg["layout"][1])
    layers = [enc.EncoderLayerWeights(hidden, ffn, tdt, seed=100 + i) for i in range(args.layers)]
    g = torch.Generator(device="cuda").manual_seed(7)
    table = (0.02 * torch.randn(vocab, hidden, device="cuda", generator=g)).to(tdt)
    pos = (0.02 * torch.randn(L, hidden, device="cuda", generator=g)).to(tdt)
    ids = torch.randint(0, vocab, (Bg, L), device="cuda", dtype=torch.int32, generator=torch.Generator(device="cuda").manual_seed(1234 + rank))
    host_ids = ids.cpu().pin_memory()
    dev_ids = torch.empty_like(ids)
    host_out = torch.empty(Bg, L, hidden, dtype=tdt).pin_memory()

    def forward(tok):
        x, _ = sfb.embedding(table, tok, pos)
        for w in layers:
            x = enc.encoder_layer(sfb, x, w, lay, H, "post", proj)
        return x

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        out = forward(ids)
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = forward(ids)
    e1.record()
    sync_all()
    eager_ms = e0.elapsed_time(e1) / args.steps
    # the forward is a few hundred short launches: captured once into a CUDA graph (on dev_ids, refreshed per step)
    dev_ids.copy_(ids)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        forward(dev_ids)
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        graph_out = forward(dev_ids)
    for _ in range(3):
        graph.replay()
    sync_all()
    sampler = ClockSampler(local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    sync_all()
    ms = e0.elapsed_time(e1) / args.steps
    out = graph_out
    # end to end: token ids from pinned host memory in, the stack's output back to the host
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        dev_ids.copy_(host_ids, non_blocking=True)
        graph.replay()
        host_out.copy_(graph_out, non_blocking=True)
    f1.record()
    sync_all()
    e2e_ms = f0.elapsed_time(f1) / args.steps
    clocks = sampler.stop() if sampler else None
    gather_ms = 0.0
    if world > 1:
        outs = torch.empty((world,) + tuple(out.shape), dtype=out.dtype, device="cuda")
        for _ in range(3):
            dist.all_gather_into_tensor(outs, out)
        sync_all()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(5):
            dist.all_gather_into_tensor(outs, out)
        g1.record()
        sync_all()
        gather_ms = g0.elapsed_time(g1) / 5
    status = sfb.device_status()
    t = torch.tensor([ms, e2e_ms, gather_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, gather_ms = (float(v) for v in t.cpu())
    if rank == 0:
        flops = args.layers * (2.0 * Bg * L * hidden * (4 * hidden + 2 * ffn) + attention_flops(dict(cfg, B=Bg), lay.blocks))
        line = {
            "metric": "encoder-stack sequences/s", "value": round(world * Bg / (ms * 1e-3), 2), "unit": "seq/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": cfg["dtype"], "data": "synthetic",
            "config": {"workload": args.config, "layers": args.layers, "B_per_gpu": Bg, "L": L, "hidden": hidden, "ffn": ffn, "heads": H,
                       "vocab": vocab, "ln": "post", "layout": cfg["layout"][0],
                       "projections": "sfb_linear (tcgen05)" if proj == "tensor" else "torch.matmul (cuBLAS)",
                       "sharding": "batch, weights replicated, no collective inside the stack",
                       "launch": "one CUDA graph replay per forward", "eager_ms_per_step": round(eager_ms, 4)},
            "tflops_per_gpu": round(flops / (ms * 1e-3) / 1e12, 1),
            "e2e": {"value": round(world * Bg / (e2e_ms * 1e-3), 2), "unit": "seq/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": Bg * L * 4, "d2h_bytes_per_step": Bg * L * hidden * table.element_size()},
            "gpu_launches": args.steps * (1 + args.layers * (7 if proj == "tensor" else 4)), "clocks": clocks, "device_status": status,   # this library's kernels per layer: QKV product, attention, 3 more products, 2 LayerNorms
        }
        if world > 1:
            line["gather_ms"] = round(gather_ms, 4)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
def run_bandwidth_kernel(args):
    """Roofline lines of the two bandwidth-bound kernels of the path (N=1): `--kernel softmax` is the
    stand-alone masked softmax (bf16 scores in, bf16 probabilities out) on the workload's layout,
    `--kernel layernorm` the fused bias + residual + LayerNorm on [B*L, H*d] rows."""
    import torch
    import __graft_entry__ as ge
    sfb = ge.load_package()
    torch.cuda.set_device(0)
    cfg = CONFIGS[args.config]
    B, H, L, d, bs = cfg["B"], cfg["H"], cfg["L"], cfg["d"], cfg["bs"]
    pk = peaks()
    flush = L2Flush(torch, args.l2_flush)
    if args.kernel == "encoder_layer":
        return run_encoder_layer(args, sfb, cfg, pk, flush)
    if args.kernel == "linear":
        return run_linear(args, sfb, cfg, pk, flush)
    if args.kernel == "csr_attention":
        tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[cfg["dtype"]]
        lay = sfb.BlockLayout.generate(getattr(sfb, cfg["layout"][0]), 1, L // bs, bs, **cfg["layout"][1])
        rowptr, colidx = sfb.csr_from_layout(lay)
        q, k, v = (torch.randn(B, L, H, d, device="cuda").to(tdt) for _ in range(3))
        fn = lambda: sfb.csr_attention(q, k, v, rowptr, colidx, 0.125)
        # what the format makes every query row gather: its keys' K and V rows (through L2), plus Q in and O out
        nbytes = int(colidx.numel()) * B * H * 2 * d * q.element_size() + 2 * q.numel() * q.element_size()
        name, unit_name = "csr_attention_split_kernel", "K and V rows gathered per query row (L2 traffic, not HBM) + Q read + O written"
    elif args.kernel == "embedding":
        tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[cfg["dtype"]]
        vocab, hidden = 30522, H * d
        table = (0.02 * torch.randn(vocab, hidden, device="cuda")).to(tdt)
        pos = (0.02 * torch.randn(L, hidden, device="cuda")).to(tdt)
        ids = torch.randint(0, vocab, (B, L), device="cuda", dtype=torch.int32)
        fn = lambda: sfb.embedding(table, ids, pos)
        nbytes = 2 * B * L * hidden * table.element_size() + B * L * 4
        name, unit_name = "embedding_kernel", "one table row read + one output row written per token (+ ids); positions stay in L2"
        lay = None
    if args.kernel in ("embedding", "csr_attention"):
        pass
    elif args.kernel == "softmax":
        lay = sfb.BlockLayout.generate(getattr(sfb, cfg["layout"][0]), cfg.get("lut_heads", 1), L // bs, bs, **cfg["layout"][1])
        x = torch.randn(B, H, lay.blocks, bs, bs, device="cuda").to(torch.bfloat16)
        fn = lambda: sfb.masked_softmax(x, lay, 0.125, torch.bfloat16)
        nbytes = x.numel() * 2 * 2
        name, unit_name = "softmax_kernel", "bf16 scores read + bf16 probabilities written"
    elif args.kernel == "softmax_grad":
        lay = sfb.BlockLayout.generate(getattr(sfb, cfg["layout"][0]), cfg.get("lut_heads", 1), L // bs, bs, **cfg["layout"][1])
        dy = torch.randn(B, H, lay.blocks, bs, bs, device="cuda").to(torch.bfloat16)
        y = torch.rand(B, H, lay.blocks, bs, bs, device="cuda").to(torch.bfloat16)
        fn = lambda: sfb.masked_softmax_grad(dy, y, lay, 0.125)
        nbytes = dy.numel() * 2 * 3
        name, unit_name = "softmax_grad_kernel", "bf16 dy and y read + bf16 dx written"
    elif args.kernel == "attention_backward":
        # the reference's five backward calls (transformer_attention_optimize.cu:924-964) on 16-bit operands, from saved probabilities
        lay = sfb.BlockLayout.generate(getattr(sfb, cfg["layout"][0]), cfg.get("lut_heads", 1), L // bs, bs, **cfg["layout"][1])
        q, k, v, do = (torch.randn(B, L, H, d, device="cuda").to(torch.bfloat16) for _ in range(4))
        pblk = sfb.fused_sddmm_softmax(q, k, lay, 0.125, torch.bfloat16)
        _ = lay.tn_lut
        blk_bytes = pblk.numel() * 2
        if args.fused_grad:
            o = sfb.bst_sgemm_xn(pblk, v, lay)
            fn = lambda: sfb.attention_backward_fused(q, k, v, pblk, o, do, lay, 0.125)
            # dV: P in; dS: P in, dS out; dK, dQ: dS in
            nbytes = 5 * blk_bytes + 10 * q.numel() * 2
            name, unit_name = "spmm_tc_kernel x3 + sddmm_tc_kernel<GRAD> + rowdot_kernel", "5 passes over the block tensors + the dense operands"
        else:
            fn = lambda: sfb.attention_backward(q, k, v, pblk, do, lay, 0.125)
            # dV: P in; dP: out; dS: dP, P in, dS out; dK, dQ: dS in -- plus each [B,L,H,d] operand once per call
            nbytes = 7 * blk_bytes + 10 * q.numel() * 2
            name, unit_name = "spmm_tc_kernel x3 + sddmm_tc_kernel + softmax_grad_kernel", "7 passes over the block tensors + the dense operands of the five calls"
    elif args.kernel == "spmm_tn":
        lay = sfb.BlockLayout.generate(getattr(sfb, cfg["layout"][0]), cfg.get("lut_heads", 1), L // bs, bs, **cfg["layout"][1])
        pblk = torch.rand(B, H, lay.blocks, bs, bs, device="cuda").to(torch.bfloat16)
        do = torch.randn(B, L, H, d, device="cuda").to(torch.bfloat16)
        fn = lambda: sfb.bst_sgemm_tn(pblk, do, lay)
        nbytes = pblk.numel() * 2 + 2 * do.numel() * 2
        name, unit_name = "spmm_tc_kernel (transposed)", "bf16 blocks read + bf16 B read once + bf16 C written"
    elif args.kernel in ("sddmm", "spmm", "fused_p"):
        tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.bfloat16}[cfg["dtype"]]
        lay = sfb.BlockLayout.generate(getattr(sfb, cfg["layout"][0]), cfg.get("lut_heads", 1), L // bs, bs, **cfg["layout"][1])
        q, k = (torch.randn(B, L, H, d, device="cuda").to(tdt) for _ in range(2))
        if args.kernel == "sddmm":
            fn = lambda: sfb.bst_sgemm_nt(q, k, lay, torch.bfloat16)
            name, unit_name = "sddmm_tc_kernel", "bf16 scores written + Q, K read once"
        elif args.kernel == "fused_p":
            fn = lambda: sfb.fused_sddmm_softmax(q, k, lay, 0.125, torch.bfloat16)
            name, unit_name = "fused_p_tc_kernel", "bf16 probabilities written + Q, K read once"
        else:
            pblk = torch.rand(B, H, lay.blocks, bs, bs, device="cuda").to(tdt)
            fn = lambda: sfb.bst_sgemm_xn(pblk, k, lay)
            name, unit_name = "spmm_tc_kernel", "16-bit probabilities read + V read once + O written"
        nbytes = B * H * lay.blocks * bs * bs * 2 + (2 if args.kernel == "sddmm" else 2) * B * L * H * d * 2
    else:
        tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[cfg["dtype"]]
        m, hidden = B * L, H * d
        x = torch.randn(m, hidden, device="cuda").to(tdt)
        r = torch.randn(m, hidden, device="cuda").to(tdt)
        bias, gain, beta = (torch.randn(hidden, device="cuda") for _ in range(3))
        fn = lambda: sfb.bias_residual_layernorm(x, bias, r, gain, beta)
        nbytes = 3 * m * hidden * x.element_size()
        name, unit_name = "bias_residual_layernorm_kernel", "x and residual read + output written"
    for _ in range(max(args.warmup, 3)):
        flush.fill_(1)
        fn()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a, b_ in ev:
        flush.fill_(1)
        a.record()
        fn()
        b_.record()
    torch.cuda.synchronize()
    ms = sum(a.elapsed_time(b_) for a, b_ in ev) / args.steps
    gbs = nbytes / (ms * 1e-3) / 1e9
    # a device-to-device copy moving the same number of bytes (half read, half written), timed the same way: what a
    # launch of this size can reach at all (the measured peak is a long copy; a short launch also pays ramp-up and tail)
    half = min(max(int(nbytes) // 2, 1 << 20), 1 << 30)   # bounded: csr_attention's bytes are gathered L2 traffic, not a buffer size
    csrc = torch.empty(half, dtype=torch.uint8, device="cuda")
    cdst = torch.empty(half, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        cdst.copy_(csrc)
    for a, b_ in ev:
        flush.fill_(1)
        a.record()
        cdst.copy_(csrc)
        b_.record()
    torch.cuda.synchronize()
    copy_ms = sum(a.elapsed_time(b_) for a, b_ in ev) / args.steps
    copy_gbs = 2.0 * half / (copy_ms * 1e-3) / 1e9
    # and a pure write of as many bytes as the copy wrote: the ceiling of a kernel that mostly writes (SDDMM, fused_p)
    for a, b_ in ev:
        flush.fill_(1)
        a.record()
        cdst.fill_(3)
        b_.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    fill_ms = sum(a.elapsed_time(b_) for a, b_ in ev) / args.steps
    fill_gbs = half / (fill_ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": args.kernel + " GB/s (algorithmic bytes)", "value": round(gbs, 1), "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5), "higher_is_better": True,
        "dtype": "bf16" if args.kernel in ("softmax", "softmax_grad", "spmm_tn", "attention_backward") else cfg["dtype"], "data": "synthetic",
        "tflops_on_kept_blocks": (round(2.0 * bs * bs * d * lay.blocks * B * H / (ms * 1e-3) / 1e12, 1)
                                  if args.kernel in ("sddmm", "spmm", "fused_p", "spmm_tn") else
                                  round(4.0 * bs * bs * d * lay.blocks * B * H / (ms * 1e-3) / 1e12, 2) if args.kernel == "csr_attention" else
                                  round(8.0 * bs * bs * d * lay.blocks * B * H / (ms * 1e-3) / 1e12, 1) if args.kernel == "attention_backward" else None),
        "config": {"workload": args.config, "kernel": name, "bytes": unit_name, "l2": flush.note},
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm"], "unit": "GB/s",
                     "frac": round(gbs / pk["hbm"], 4), "traffic": None, "peak_source": pk["source"] + " copy bandwidth",
                     "algorithmic_bytes": nbytes,
                     "copy_of_same_bytes": {"gbs": round(copy_gbs, 1), "ms": round(copy_ms, 5),
                                            "frac_of_it": round(gbs / copy_gbs, 4)},
                     "fill_gbs": round(fill_gbs, 1)},
        "gpu_launches": args.steps * (5 if args.kernel == "attention_backward" else 1), "clocks": clocks}), flush=True)


def run_linear(args, sfb, cfg, pk, flush):
    """The dense projections of one encoder layer at the workload's shape on the tcgen05 kernel (N=1): QKV as one
    [hidden, 3 hidden] product, the output projection, FFN up (with GELU) and FFN down; the GEMM library's time on
    the same products is printed beside it."""
    import torch
    B, H, L, d = cfg["B"], cfg["H"], cfg["L"], cfg["d"]
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.bfloat16}[cfg["dtype"]]
    hidden, ffn, m = H * d, 4 * H * d, B * L
    shapes = [("qkv", hidden, 3 * hidden, 0), ("out", hidden, hidden, 0), ("ffn_up_gelu", hidden, ffn, 1), ("ffn_down", ffn, hidden, 0),
              ("logits_tied", hidden, 30528, -1)]   # the vocabulary of 30522 padded to a multiple of 16; not part of the layer total
    res, total_ms, total_lib, flops = {}, 0.0, 0.0, 0.0
    sampler = ClockSampler(0)
    for name, k, n, act in shapes:
        x = torch.randn(m, k, device="cuda").to(tdt)
        if act < 0:
            wt = (0.02 * torch.randn(n, k, device="cuda")).to(tdt)
            out = torch.empty(m, n, device="cuda", dtype=tdt)
            ours = lambda: sfb.linear_nt(x, wt, None, 0, out=out)
            libf = lambda: torch.matmul(x, wt.t(), out=out)
        else:
            w = (0.02 * torch.randn(k, n, device="cuda")).to(tdt)
            b = torch.randn(n, device="cuda")
            ours = lambda: sfb.linear(x, w, b, act)
            if act:
                libf = lambda: torch.nn.functional.gelu(torch.addmm(b.to(tdt), x, w))
            else:
                libf = lambda: torch.addmm(b.to(tdt), x, w)
        t = []
        for fn in (ours, libf):
            for _ in range(max(args.warmup, 3)):
                fn()
            torch.cuda.synchronize()
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
            for a, b_ in ev:
                flush.fill_(1)
                a.record()
                fn()
                b_.record()
            torch.cuda.synchronize()
            t.append(sum(a.elapsed_time(b_) for a, b_ in ev) / args.steps)
        f = 2.0 * m * n * k
        res[name] = {"m": m, "n": n, "k": k, "ms": round(t[0], 4), "tflops": round(f / (t[0] * 1e-3) / 1e12, 1),
                     "library_ms": round(t[1], 4), "library_tflops": round(f / (t[1] * 1e-3) / 1e12, 1)}
        if act >= 0:
            total_ms += t[0]
            total_lib += t[1]
            flops += f
    clocks = sampler.stop()
    tf = flops / (total_ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "projection TFLOP/s", "value": round(tf, 1), "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(total_ms, 4), "higher_is_better": True, "dtype": cfg["dtype"],
        "data": "synthetic",
        "config": {"workload": args.config, "kernel": "linear_tc_kernel", "products": res, "library": "torch.addmm (+ gelu) on cuBLAS",
                   "library_ms": round(total_lib, 4), "l2": flush.note},
        "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": pk["tensor"], "unit": "TFLOP/s", "frac": round(tf / pk["tensor"], 4),
                     "traffic": None, "peak_source": pk["source"] + " cuBLAS bf16 burst"},
        "gpu_launches": args.steps * 4, "clocks": clocks}), flush=True)


def run_encoder_layer(args, sfb, cfg, pk, flush):
    """Sequences per second of one encoder layer (post-LN, GELU FFN of 4 x hidden) at the workload's shape:
    projections by the GEMM library, attention / LayerNorm / GELU by this library (N=1)."""
    import importlib.util
    import torch
    spec = importlib.util.spec_from_file_location("sfb_encoder", os.path.join(ROOT, "sf-bert_b200", "encoder.py"))
    enc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(enc)
    B, H, L, d, bs = cfg["B"], cfg["H"], cfg["L"], cfg["d"], cfg["bs"]
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[cfg["dtype"]]
    hidden, ffn = H * d, 4 * H * d
    lay = sfb.BlockLayout.generate(getattr(sfb, cfg["layout"][0]), cfg.get("lut_heads", 1), L // bs, bs, **cfg["layout"][1])
    w = enc.EncoderLayerWeights(hidden, ffn, tdt, seed=1)
    x = torch.randn(B, L, hidden, device="cuda").to(tdt)
    proj = "tensor" if args.projections == "tensor" and tdt != torch.float32 else "library"
    fn = lambda: enc.encoder_layer(sfb, x, w, lay, H, "post", proj)
    for _ in range(max(args.warmup, 3)):
        fn()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a, b_ in ev:
        flush.fill_(1)
        a.record()
        fn()
        b_.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = sum(a.elapsed_time(b_) for a, b_ in ev) / args.steps
    gemm_flops = 2.0 * B * L * hidden * (4 * hidden + 2 * ffn)
    attn_flops = attention_flops(cfg, lay.blocks)
    print(json.dumps({
        "metric": "encoder-layer sequences/s", "value": round(B / (ms * 1e-3), 2), "unit": "seq/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4), "higher_is_better": True,
        "dtype": cfg["dtype"], "data": "synthetic",
        "config": {"workload": args.config, "B": B, "L": L, "hidden": hidden, "ffn": ffn, "heads": H, "ln": "post",
                   "projections": "sfb_linear (tcgen05, bias/GELU in the epilogue)" if proj == "tensor" else "torch.matmul (cuBLAS)",
                   "l2": flush.note},
        "tflops_total": round((gemm_flops + attn_flops) / (ms * 1e-3) / 1e12, 1),
        "gpu_launches": args.steps * (7 if proj == "tensor" else 4), "clocks": clocks}), flush=True)



# ------------------------------------------------------------------------------------------------
def run_dropin(args):
    """The reference's own call signature on the reference's own micro-benchmark shape (stride_fusion_test.cu:19-24:
    B=32, H=4, d=128, 32x32 blocks, L=1024, fp32 Q/K/V, its sawtooth "stride" layout): the operators a program that
    includes include/blocksparse.h / include/fusion_blocksparse.h reaches (their bodies are one-line forwarders to the
    C ABI entry points called here with the same arguments) timed beside the reference's own unfused GPU operators
    compiled for sm_100a (oracle/_ref/libsfb_ref_gpu.so) on the same inputs.  fp32 operands run on this library's
    CUDA-core kernels (tensor-core arithmetic cannot meet fp32 parity); the reference's fused kernels spin on global
    flags without a bound and are not run."""
    import torch
    import __graft_entry__ as ge
    sfb = ge.load_package()
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    torch.cuda.set_device(0)
    B, H, L, d, bs = 32, 4, 1024, 128, 32
    nb = L // bs
    lay = sfb.BlockLayout.generate(sfb.LAYOUT_SAWTOOTH, 1, nb, bs, p0=8)
    gen = torch.Generator(device="cuda").manual_seed(1234)
    q, k, v = (torch.randn(B, L, H, d, device="cuda", generator=gen) for _ in range(3))
    scale = 1.0 / d ** 0.5
    flush = L2Flush(torch, args.l2_flush)

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for a, b_ in ev:
            flush.fill_(1)
            a.record()
            fn()
            b_.record()
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b_) for a, b_ in ev) / args.steps

    def trio():
        s_ = sfb.bst_sgemm_nt(q, k, lay, torch.bfloat16)
        p_ = sfb.masked_softmax(s_, lay, scale, torch.bfloat16)
        return sfb.bst_sgemm_xn(p_, v, lay)

    ours = {
        "fusion_attention2<float,float2> (SDDMM + softmax, fp32 P out)": timed(lambda: sfb.fused_sddmm_softmax(q, k, lay, scale, torch.float32)),
        "bst_sgemm_nt + BlocksparseMaskedSoftmax<bhalf> + bst_sgemm_xn": timed(trio),
        "fusion_attention (SDDMM + softmax + SpMM in one launch)": timed(lambda: sfb.fused_attention(q, k, v, lay, scale)),
    }
    ref_ms = None
    if O.ref_gpu() is not None:
        ref = O.RefGpuAttention(O.layout("sawtooth", 1, nb, chunks=8))
        ref.alloc(q)
        ref_ms = timed(lambda: ref.launch(q, k, v, scale))
        got = sfb.fused_attention(q, k, v, lay, scale)
        err = float((got - ref.o).abs().max() / ref.o.abs().max())
    flops = 4.0 * bs * bs * d * lay.blocks * B * H
    best = ours["fusion_attention (SDDMM + softmax + SpMM in one launch)"]
    print(json.dumps({
        "metric": "block-sparse attention TFLOP/s on nonzero blocks", "value": round(flops / (best * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(best, 4), "higher_is_better": True,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "reference micro-benchmark shape (stride_fusion_test.cu:19-24)", "B": B, "H": H, "L": L, "d": d, "block": bs,
                   "layout": "LAYOUT_SAWTOOTH chunks=8", "nnz_blocks_per_head": lay.blocks, "l2": flush.note},
        "ours_ms": {k_: round(v_, 4) for k_, v_ in ours.items()},
        "reference_gpu": None if ref_ms is None else {
            "ms_per_step": round(ref_ms, 4), "value": round(flops / (ref_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
            "what": "reference bst_sgemm_nt + BlocksparseMaskedSoftmax<bhalf> + bst_sgemm_xn(NN) compiled for sm_100a, same inputs",
            "max_rel_diff_of_O": round(err, 5)},
        "gpu_launches": args.steps * 5}), flush=True)

# ------------------------------------------------------------------------------------------------
def cpu_reference_sample(cfg, budget_s, steps):
    """Times the reference's CPU attention operators (multiheadmatmulNT -> softmax -> multiheadmatmulNN,
    transformer_inference_part.cpp:219-224) on B' = host threads batches x 1 head, at the longest
    sequence length whose estimated time fits the budget.  The reference parallelises over the batch only."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    R = O.ref()
    kind = "reference"
    # all the host threads this process may use: launchers such as torchrun hand their children OMP_NUM_THREADS=1
    host = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    if R is not None:
        R.ref_set_num_threads(host)
    O.lib().orc_set_num_threads(host)
    threads = R.ref_num_threads() if R is not None else O.lib().orc_num_threads()
    if R is None:
        kind = "port"
    d, bs = cfg["d"], cfg["bs"]
    Bs = max(1, min(threads, 16))

    def one(Ls, reps):
        nb = Ls // bs
        luts = O.lut_build(O.layout(cfg["oracle"][0], 1, nb, **cfg["oracle"][1]))
        q, k, v = (O.fill_normal((Bs, Ls, 1, d), 50 + i) for i in range(3))
        times = []
        for _ in range(reps):
            t0 = time.perf_counter()
            if R is not None:
                O.ref_dense_causal_attention(q, k, v, np.float32(1.0 / d ** 0.5))
            else:
                O.attention(q, k, v, luts, bs, np.float32(1.0 / d ** 0.5), want=("o",))
            times.append(time.perf_counter() - t0)
        flops = 4.0 * bs * bs * d * luts["blocks"] * Bs
        return times, flops, luts["blocks"]

    cal, _, _ = one(512, 1)
    Ls = 512
    for cand in (cfg["L"], cfg["L"] // 2, cfg["L"] // 4, cfg["L"] // 8):
        if cand >= 512 and cal[0] * (cand / 512.0) ** 2 <= budget_s / max(steps, 1):
            Ls = cand
            break
    times, flops, blocks = one(Ls, steps)
    best = sum(times) / len(times)
    return {"value": flops / best / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": kind,
            "sample": "%d batches x 1 head, L=%d of %d, d=%d: reference multiheadmatmulNT + softmax + multiheadmatmulNN "
                      "(dense causal, OpenMP over the batch), flops counted on the %d kept blocks of the %s layout at that "
                      "length; %.2f s per pass" % (Bs, Ls, cfg["L"], d, blocks, cfg["oracle"][0], best),
            "seconds_per_pass": best, "L_sample": Ls}


def reference_gpu_sample(cfg, steps, warmup):
    """Times the reference's own unfused GPU operators on this GPU: bst_sgemm_nt -> BlocksparseMaskedSoftmax ->
    bst_sgemm_xn (the three launches of transformer_attention_optimize.cu:728,738,748), compiled for sm_100a from the
    reference header.  Its matmuls exist for 32x32 blocks only, so the workload's layout is split into 32x32 blocks:
    the same element mask, the same attention, four times the block count.  fp32 activations, bf16 scores and
    probabilities, as the reference stores them.  Returns None without a GPU or without the prebuilt library.
    The reference's fused kernels spin on global flags without a bound and are not run."""
    try:
        import torch
    except ImportError:
        return None
    if not torch.cuda.is_available():
        return None
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    if O.ref_gpu() is None:
        return None
    B, H, L, d, bs = cfg["B"], cfg["H"], cfg["L"], cfg["d"], cfg["bs"]
    lay = O.layout(cfg["oracle"][0], cfg.get("lut_heads", 1), L // bs, **cfg["oracle"][1])
    kept = int(lay[0].sum())
    if bs != 32:
        lay = O.split_layout(lay, bs // 32)
    ref = O.RefGpuAttention(lay)
    g = torch.Generator(device="cuda").manual_seed(1234)
    q, k, v = (torch.randn(B, L, H, d, device="cuda", generator=g) for _ in range(3))
    ref.alloc(q)
    scale = 1.0 / d ** 0.5
    for _ in range(max(warmup, 3)):
        ref.launch(q, k, v, scale)
    torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(max(steps, 1))]
    for marks in ev:
        ref.launch(q, k, v, scale, marks)
    torch.cuda.synchronize()
    ms = statistics.mean(m[0].elapsed_time(m[3]) for m in ev)
    per_launch = [statistics.mean(m[i].elapsed_time(m[i + 1]) for m in ev) for i in range(3)]
    flops = 4.0 * bs * bs * d * kept * B * H
    finite = bool(torch.isfinite(ref.o).all())
    # the reference's five backward calls (transformer_attention_optimize.cu:924-964) on the same 32x32 layout, from the
    # probabilities its forward just wrote: dV = P^T dO, dP = dO V^T, dS = softmax gradient, dK = dS^T Q, dQ = dS K
    import ctypes as C
    G_ = O.ref_gpu()
    tn = O.lut_build_tn(lay)
    tn_lut = torch.from_numpy(tn["tn"].view("int32")).cuda()
    do = torch.randn(B, L, H, d, device="cuda", generator=g)
    dv, dk, dq = (torch.empty_like(q) for _ in range(3))
    dp, ds = torch.empty_like(ref.s), torch.empty_like(ref.s)
    nb32, heads32 = ref.nb, ref.heads
    u, vp = C.c_uint32, lambda t: C.c_void_p(t.data_ptr())

    def backward(marks=None):
        st_ = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        common = (u(32), u(ref.blocks), u(B), u(nb32), u(nb32), u(H), u(d), u(heads32))
        rcs = []
        if marks: marks[0].record()
        rcs.append(G_.ref_gpu_bst_sgemm_tn(st_, vp(tn_lut), vp(ref.p), vp(do), vp(dv), *common, u(ref.blocks + nb32), u(tn["tn_max"])))
        rcs.append(G_.ref_gpu_bst_sgemm_nt(st_, vp(ref.nt), vp(do), vp(v), vp(dp), *common, u(ref.blocks)))
        rcs.append(G_.ref_gpu_masked_softmax_grad(st_, vp(ref.nn), vp(dp), vp(ref.p), vp(ds), u(32), u(ref.blocks), u(B), u(H), u(nb32),
                                                  u(heads32), u(ref.blocks + nb32), u(ref.nn_max), C.c_float(scale)))
        rcs.append(G_.ref_gpu_bst_sgemm_tn(st_, vp(tn_lut), vp(ds), vp(q), vp(dk), *common, u(ref.blocks + nb32), u(tn["tn_max"])))
        rcs.append(G_.ref_gpu_bst_sgemm_nn(st_, vp(ref.nn), vp(ds), vp(k), vp(dq), *common, u(ref.blocks + nb32), u(ref.nn_max)))
        if marks: marks[1].record()
        assert not any(rcs), rcs
    for _ in range(3):
        backward()
    torch.cuda.synchronize()
    for m_ in ev:
        backward(m_)
    torch.cuda.synchronize()
    bwd_ms = statistics.mean(m_[0].elapsed_time(m_[1]) for m_ in ev)
    bwd_finite = bool(torch.isfinite(dq).all() and torch.isfinite(dk).all() and torch.isfinite(dv).all())
    softmax64 = None
    if bs == 64:
        # the reference's softmax (not its matmuls) also exists for 64x64 blocks: the workload's own layout, bf16 in and out
        import ctypes as C
        lay64 = O.layout(cfg["oracle"][0], cfg.get("lut_heads", 1), L // bs, **cfg["oracle"][1])
        luts = O.lut_build(lay64)
        nn = torch.from_numpy(luts["nn"].view("int32")).cuda()
        xs = torch.randn(B, H, luts["blocks"], 64, 64, device="cuda", generator=g).to(torch.bfloat16)
        ys = torch.empty_like(xs)
        u, vp = C.c_uint32, lambda t: C.c_void_p(t.data_ptr())

        def soft():
            rc = O.ref_gpu().ref_gpu_masked_softmax(C.c_void_p(torch.cuda.current_stream().cuda_stream), vp(nn), None, vp(xs), vp(ys),
                                                    C.c_int(0), u(64), u(luts["blocks"]), u(B), u(H), u(L // bs), u(lay64.shape[0]),
                                                    u(luts["blocks"] + L // bs), u(luts["nn_max"]), u(1), C.c_float(scale))
            assert rc == 0, rc
        for _ in range(3):
            soft()
        torch.cuda.synchronize()
        for m_ in ev:
            m_[0].record()
            soft()
            m_[1].record()
        torch.cuda.synchronize()
        sm_ms = statistics.mean(m_[0].elapsed_time(m_[1]) for m_ in ev)
        softmax64 = {"ms": round(sm_ms, 4), "gbs": round(xs.numel() * 4 / (sm_ms * 1e-3) / 1e9, 1),
                     "what": "reference BlocksparseMaskedSoftmax<bhalf> on the workload's own 64x64 layout, bf16 in and out"}
    return {"value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "launches_per_step": 3,
            "ms_sddmm_softmax_spmm": [round(x, 4) for x in per_launch], "blocks_32x32_per_head": ref.blocks, "finite": finite, "softmax_block64": softmax64,
            "backward": {"ms_per_step": round(bwd_ms, 4), "launches_per_step": 5, "finite": bwd_finite,
                         "what": "reference bst_sgemm_xn(TN) + bst_sgemm_nt + BlocksparseMaskedSoftmaxGrad<bhalf> + bst_sgemm_xn(TN) + "
                                 "bst_sgemm_xn(NN) on the same 32x32 layout, fp32 activations, bf16 block tensors"},
            "what": "reference bst_sgemm_nt + BlocksparseMaskedSoftmax<bhalf> + bst_sgemm_xn(NN) on this GPU, fp32 "
                    "activations, bf16 scores, the %s layout split into 32x32 blocks, inputs larger than L2, CUDA events"
                    % cfg["oracle"][0]}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = CONFIGS[args.config]
    n = max(args.steps + args.warmup, 1)
    res = cpu_reference_sample(cfg, budget_s=150.0, steps=n)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    line = {
        "impl": "reference", "metric": "block-sparse attention TFLOP/s on nonzero blocks", "value": res["value"],
        "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": res["seconds_per_pass"] * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.config, "L": cfg["L"], "d": cfg["d"], "block": cfg["bs"], "layout": cfg["layout"][0]},
        "cpu_baseline": {"value": res["value"], "unit": "TFLOP/s", "cores": res["cores"], "kind": res["kind"], "sample": res["sample"]},
        "e2e": {"value": res["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    gpu = reference_gpu_sample(cfg, args.steps, args.warmup)
    if gpu is not None:
        line["reference_gpu"] = gpu
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="stride_bertbase", choices=sorted(CONFIGS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the encoder-layer / encoder-stack / strong-scaling legs of the default line")
    ap.add_argument("--kernel", default="fused", choices=["fused", "softmax", "layernorm", "sddmm", "spmm", "fused_p", "encoder_layer", "softmax_grad", "spmm_tn", "linear", "embedding", "encoder_stack", "csr_attention", "attention_backward", "dropin"],
                    help="fused = the headline fused attention; softmax / layernorm = the bandwidth kernels (N=1)")
    ap.add_argument("--projections", default="tensor", choices=["tensor", "library"],
                    help="--kernel encoder_layer: the layer's GEMMs on this library's tcgen05 kernel or on the GEMM library")
    ap.add_argument("--fused-grad", action="store_true", help="--kernel attention_backward: dP and dS in one launch (sfb_fused_sddmm_softmax_grad)")
    ap.add_argument("--l2-flush", default="write_read", choices=["write_read", "write"],
                    help="what runs between timed steps: 256 MB written and 256 MB read (cold, clean L2), or the write alone")
    ap.add_argument("--layers", type=int, default=24, help="--kernel encoder_stack: number of encoder layers")
    a = ap.parse_args()
    if a.impl == "reference":
        run_reference(a)
    elif a.kernel == "encoder_stack":
        run_encoder_stack(a)
    elif a.kernel == "dropin":
        run_dropin(a)
    elif a.kernel != "fused":
        run_bandwidth_kernel(a)
    else:
        run_ours(a)
    if a.impl != "reference":
        # a kernel that gave up on a bounded wait leaves its code in the library's status word: the numbers above are
        # then not measurements, and the run says so with its exit code (every rank looks at its own device)
        import __graft_entry__ as ge
        status = ge.load_package().device_status()
        if status:
            print("bench.py: device status word 0x%08x (a kernel gave up on a bounded wait): results invalid" % status, file=sys.stderr)
            sys.exit(3)
