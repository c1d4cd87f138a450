#!/usr/bin/env python
"""Benchmark of the KAD-Conv inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4|c0|c1|c2|c4-kernel|conv3x3|gemm1x1] [--impl ours|reference]

Prints ONE JSON line on stdout (rank 0; everything else goes to stderr). Workloads (BASELINE.json configs):
  c4  (default) KAD-CNet-S detector, fp16, 64 uint8 3x800x800 synthetic images per step sharded over the ranks:
      backbone + neck + head + decode + NMS. `value` = images/s with the images resident in HBM; `e2e` = the same
      through the public Python API from pinned host images, detections read back, both copies inside the timed
      region; `roofline` = the kernel with the largest share of the forward timed alone; `kadconv_op` = the c1
      measurement below, taken in the same run (the second half of the metric: op microseconds + % of roofline).
  c0  KADConv(64) on x[2,64,80,80] fp32 through the module API: microseconds per forward next to the plain module on the GPU and the CPU.
  c1  KAD-Conv operator alone: DSC 256->256, [16,256,100,100] fp16, offsets N(0,2) px, mask given (gather +
      tcgen05 implicit GEMM). One step = one pass over the batch of 16 feature maps.
  c2  bf16 KADConv(128) at 200x200 + avg-pool + 1x1 GEMM+SiLU + SE, with a per-kernel-group table.
  c4-kernel  the detector's dominant kernel alone (small enough to profile).
  gemm1x1  the detector's 1x1 GEMM + bias + SiLU shapes on the tcgen05 GEMM kernel, GB/s against the measured HBM peak.
  conv3x3  the detector's 3x3 convolution shapes: this package's tcgen05 kernel next to the library path (table in the line).
`--impl reference` times the plain PyTorch modules + torchvision (what the reference's raw backend executes) on the
host cores on a bounded sample of the same workload.
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
for p in (ROOT, ROOT / 'kad-conv_b200'):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

import torch  # noqa: E402

C1 = dict(B=16, C=256, H=100, W=100)
C1_FLOPS = 2.0 * C1['B'] * C1['H'] * C1['W'] * C1['C'] * 9 * C1['C']                    # 188.74 GFLOP
C1_BYTES = 2.0 * (C1['B'] * C1['H'] * C1['W'] * (2 * C1['C'] + 27) + 9 * C1['C'] * C1['C'])  # 173.66 MB
NCU_TRAFFIC = {'c1': 129.8e6, 'c4_dsc_mma': 38.5e6}   # c4_dsc_mma: reads only; the 15.4 MB written were still in L2 when the counters stopped   # DRAM bytes per launch from the committed ncu summary (profiles/), filled below
NCU_ISSUE = {'c4_dsc_mma': 0.48}        # issue slots busy, from the committed ncu summary of that kernel
NCU_LSU_PIPE = {'c4_dsc_mma': 0.71}     # L1 / shared-memory data pipe (LSU wavefronts) busy, same summary
FALLBACK_PEAKS = {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0}


def peaks():
    f = ROOT / 'MEASURED_PEAKS.json'
    if f.exists():
        d = json.loads(f.read_text())
        d['_source'] = 'measured'
        return d
    d = dict(FALLBACK_PEAKS)
    d['_source'] = 'fallback'
    return d


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    Q = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
         'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.index, self.proc, self.lines, self.t_begin = index, None, [], 0.0

    def start(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.index), f'--query-gpu={self.Q}', '--format=csv,noheader,nounits',
                                          '-lms', '100'], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def begin(self):
        """The timed region starts now: only samples taken from here on count. (The sampler itself is started before the warm-up,
        so that nvidia-smi's start-up, which attaches to every GPU of the box, is over by then.)"""
        deadline = time.time() + 5.0
        while self.proc is not None and not self.lines and time.time() < deadline:      # its first line means the start-up is over
            time.sleep(0.01)
        self.t_begin = time.time()

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        t_end = time.time()
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        inside = [ln for ts, ln in self.lines if self.t_begin - 0.05 <= ts <= t_end + 0.12]
        for ln in (inside or [ln for _, ln in self.lines[-3:]]):
            f = [v.strip() for v in ln.split(',')]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith('active'):
                    reasons.add(n)
        return {'sm_mhz': statistics.median(sm) if sm else None, 'sm_max_mhz': max(mx) if mx else None,
                'samples': len(sm), 'reasons': sorted(reasons)}


def dist_setup(n):
    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    local = int(os.environ.get('LOCAL_RANK', 0))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        backend = 'nccl' if torch.cuda.is_available() else 'gloo'
        if backend == 'nccl':
            torch.cuda.set_device(local)
        dist.init_process_group(backend, **({'device_id': torch.device('cuda', local)} if backend == 'nccl' else {}))
    return rank, world, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def max_over_ranks(v, world, device):
    if world == 1:
        return v
    import torch.distributed as dist
    t = torch.tensor([v], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def cpu_info():
    model = 'unknown'
    try:
        for ln in open('/proc/cpuinfo'):
            if ln.startswith('model name'):
                model = ln.split(':', 1)[1].strip(); break
    except OSError:
        pass
    return model, os.cpu_count()


# ------------------------------------------------------------------------------------------- C1
def c1_inputs(device, seed, dtype=torch.float16):
    g = torch.Generator(device='cpu').manual_seed(seed)
    B, C, H, W = C1['B'], C1['C'], C1['H'], C1['W']
    x = torch.randn((B, C, H, W), generator=g).to(dtype)
    off = (2.0 * torch.randn((B, 18, H, W), generator=g)).to(dtype)
    msk = torch.sigmoid(torch.randn((B, 9, H, W), generator=g)).to(dtype)
    w = ((torch.rand((C, C, 3, 3), generator=g) * 2 - 1) / 48.0).to(dtype)
    b = torch.zeros(C)
    return x, off, msk, w, b


def c1_cpu_step(x, off, msk, w, b, i):
    """One feature map of the c1 batch through torchvision.ops.deform_conv2d (what DSC.forward calls in the reference), fp32, all host cores."""
    import torchvision
    t0 = time.perf_counter()
    with torch.no_grad():
        torchvision.ops.deform_conv2d(x[i:i + 1], off[i:i + 1], w, b, stride=1, padding=1, mask=msk[i:i + 1])
    return time.perf_counter() - t0


def c1_cpu_inputs():
    torch.set_num_threads(os.cpu_count() or 1)
    x, off, msk, w, b = c1_inputs('cpu', 0)
    return x.float(), off.float(), msk.float(), w.float(), b


def c1_cpu_sample(n_maps=5, warmup=1):
    """Median over `n_maps` single-map steps; returns (feature maps/s, n, seconds)."""
    t = c1_cpu_inputs()
    for i in range(warmup):
        c1_cpu_step(*t, i)
    ts = [c1_cpu_step(*t, (warmup + i) % C1['B']) for i in range(n_maps)]
    return 1.0 / statistics.median(ts), n_maps, sum(ts)


def c1_torch_gpu_sample(device, iters=5):
    """torchvision.ops.deform_conv2d on the same GPU in fp16 (NCHW, the library's im2col + GEMM): the call the reference makes."""
    import torchvision
    x, off, msk, w, b = (t.to(device) for t in c1_inputs(device, 0))
    b = b.half()

    def once():
        with torch.no_grad():
            return torchvision.ops.deform_conv2d(x, off, w, b, stride=1, padding=1, mask=msk)
    for _ in range(2):
        once()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        once()
    e1.record(); torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / iters * 1e3
    return {'us_per_op': us, 'tflops': C1_FLOPS / us / 1e6, 'dtype': 'f16', 'what': 'torchvision.ops.deform_conv2d on the same GPU (library kernels)'}


def run_c1(args, rank, world, local):
    from kadconv import ops
    import kadconv.functional as KF
    device = torch.device('cuda', local)
    torch.cuda.set_device(device)
    dtype = torch.float16
    # two input sets, alternated, so that no step finds its inputs in L2 (each set is 174 MB > 126 MB L2 anyway)
    sets = []
    for s in range(2):
        x, off, msk, w, b = c1_inputs(device, s)
        sets.append(dict(x=ops.to_nhwc(x.to(device)), off=ops.to_nhwc(off.to(device)), msk=ops.to_nhwc(msk.to(device)),
                         host=(x.pin_memory(), off.pin_memory(), msk.pin_memory())))
    wdev = w.to(device)
    wp = ops.pack_dsc_weight_tc(wdev.float(), dtype)
    stream = torch.cuda.current_stream()

    def step(i):
        s = sets[i & 1]
        return ops.dsc_forward(s['x'], wp, s['off'], s['msk'], path=ops.PATH_TC, cout=C1['C'])

    sampler = ClockSampler(local); sampler.start()
    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize(); ops.check_status(device)
    barrier(world); torch.cuda.synchronize()
    sampler.begin()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(args.steps):
        evs[i][0].record(stream); step(i); evs[i][1].record(stream)
    e1.record(stream)
    torch.cuda.synchronize(); barrier(world)
    clocks = sampler.stop()
    ops.check_status(device)
    ms_total = max_over_ranks(e0.elapsed_time(e1), world, device)
    kern_ms = statistics.mean(a.elapsed_time(b) for a, b in evs)

    # end to end through the public op (NCHW host tensors in, NCHW host tensor out)
    weight_mod = KF.PackedDeformWeight(wdev.float(), dtype)
    out_host = torch.empty((C1['B'], C1['C'], C1['H'], C1['W']), dtype=dtype).pin_memory()

    def e2e_step(i):
        hx, ho, hm = sets[i & 1]['host']
        y = KF.deform_conv2d(hx.to(device, non_blocking=True), ho.to(device, non_blocking=True), weight_mod, None,
                             mask=hm.to(device, non_blocking=True))
        out_host.copy_(y, non_blocking=True)

    n_e2e = 0 if args.profile else max(2, args.steps)
    for i in range(2 if n_e2e else 0):
        e2e_step(i)
    torch.cuda.synchronize(); barrier(world)
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    for i in range(n_e2e):
        e2e_step(i)
    f1.record(stream)
    torch.cuda.synchronize(); barrier(world)
    e2e_ms = max_over_ranks(f0.elapsed_time(f1), world, device) / max(n_e2e, 1)
    ops.check_status(device)
    h2d = sum(t.numel() * t.element_size() for t in sets[0]['host'])
    d2h = out_host.numel() * out_host.element_size()

    pk = peaks()
    achieved = C1_FLOPS / (kern_ms * 1e-3) / 1e12
    res = {
        'metric': 'KAD-Conv op (DSC 256->256 @100x100 fp16) feature maps/s', 'value': world * C1['B'] * args.steps / (ms_total * 1e-3),
        'unit': 'images/s', 'n_gpus': world, 'steps': args.steps, 'warmup': max(args.warmup, 3),
        'ms_per_step': ms_total / args.steps, 'us_per_op': kern_ms * 1e3, 'higher_is_better': True, 'scaling': 'weak',
        'vs_baseline': None, 'dtype': 'f16', 'data': 'synthetic',
        'config': {'workload': C1_WORKLOAD, 'l2': C1_L2},
        'run': {'per_gpu_batch': C1['B'], 'l2': 'two 174 MB input sets alternated (each larger than the 126 MB L2)', 'layout': 'NHWC in HBM'},
        'roofline': {'bound': 'tensor', 'achieved': achieved, 'peak': pk['bf16_tflops'], 'unit': 'TFLOP/s',
                     'frac': achieved / pk['bf16_tflops'], 'traffic': NCU_TRAFFIC['c1'], 'peak_source': pk['_source'] + ' (burst)',
                     'kernel': 'dsc_tc_kernel', 'flops_per_launch': C1_FLOPS, 'algorithmic_bytes': C1_BYTES,
                     'hbm_frac_of_peak': C1_BYTES / (kern_ms * 1e-3) / 1e9 / pk['hbm_gbs']},
        'e2e': None if args.profile else {'value': world * C1['B'] / (e2e_ms * 1e-3), 'unit': 'images/s', 'h2d_bytes_per_step': h2d,
                                           'd2h_bytes_per_step': d2h, 'ms_per_step': e2e_ms},
        'gpu_launches': args.steps * 1,
        'clocks': clocks,
    }
    return res



# ------------------------------------------------------------------------------------------- C4
C4 = dict(images=64, H=800, W=800, mb=8, conf=0.001, iou=0.65, max_det=300)
C4_GFLOP_PER_IMAGE = 38.9          # 2*MAC of the fused model at 800x800 (72 % 3x3 conv, 22 % 1x1 conv, 1.9 % DSC GEMM)
C4_MIN_BYTES_PER_IMAGE = 0.35e9    # sum of conv inputs + outputs in fp16: the activation traffic floor


C4_WORKLOAD = ('c4: KAD-CNet-S (dior_s_base graph, 20 classes, seeded synthetic weights), batches of uint8 3x800x800 images, 64 per GPU and step, '
               'sharded by batch over the ranks (no collective, host gather of the detections): backbone + neck + head + decode + NMS '
               '(conf 0.001, IoU 0.65, max_det 300)')
C1_WORKLOAD = 'c1: DSC 256->256, x[16,256,100,100] fp16, offsets N(0,2) px, mask sigmoid(N(0,1)), W U(+-1/48)'
# how consecutive timed iterations are kept from finding their inputs in the 126 MB L2 (the same statement on both arms)
C4_L2 = 'inputs larger than L2: one step reads 123 MB of images and its activations (about 0.35 GB per image) never fit the 126 MB L2'
C1_L2 = 'inputs larger than L2: two input sets of 173 MB each are alternated between timed iterations'


def c4_images(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 256, (n, 3, C4['H'], C4['W']), dtype=torch.uint8, generator=g)


def c4_dominant_kernel(device, mb, stream, n=20, variant='tensor'):
    """The kernel with the largest share of the detector forward, timed alone with CUDA events: the deformable convolution of a
    KAD-Conv branch with the offset convolution fused in, at the detector's largest KAD-Conv shape (stride 8: 100x100, 12
    channels). variant='tensor' (what the layer call launches by default) reads the float32 LCSA mask tensor; variant='inline'
    evaluates the mask in-kernel (KadLayerArgs.scheme = 3). Two input sets are alternated.
    """
    from kadconv import ops
    B, H, W, c = mb, 100, 100, 12
    Cp = (c + 3) & ~3
    g = torch.Generator(device=device).manual_seed(1)
    r = lambda *shape, s=1.0: torch.randn(shape, device=device, generator=g) * s
    sets = []
    for _ in range(2):
        x = r(B, H, W, c).half()
        if variant == 'inline':
            xf = x.float()
            extra = dict(rowmean=xf.mean(2).contiguous(), A=r(B, W, Cp, s=0.3), Sm=r(W, Cp, s=0.3), w2=r(c, 11, s=0.3), b2=r(c, s=0.1), w3=r(9, c, s=0.3), b3=r(9, s=0.1))
        else:
            extra = torch.sigmoid(r(B, H, W, 9))
        sets.append((x, extra))
    w = ops.pack_dsc_weight_simt((torch.rand((c, c, 3, 3), device=device, generator=g) * 2 - 1) / (3 * c ** 0.5))
    wo = ops.pack_dsc_weight_simt((torch.rand((18, c, 3, 3), device=device, generator=g) * 2 - 1) / (3 * c ** 0.5))
    frags = ops.pack_dsc_mma_frags(w, wo, torch.float16)      # as the layer call passes them: packed once, copied by every block
    bo = torch.zeros(18, device=device)

    def launch(i):
        x, extra = sets[i & 1]
        if variant == 'inline':
            return ops.dsc_forward(x, w, None, None, act=ops.ACT_RELU, path=ops.PATH_MMA, want_gap=True, offset_weight=wo, offset_bias=bo, lcsa_inline=extra)
        return ops.dsc_forward(x, w, None, extra, act=ops.ACT_RELU, path=ops.PATH_MMA, want_gap=True, offset_weight=wo, offset_bias=bo, mma_frags=frags)

    for i in range(3):
        launch(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(n):
        launch(i)
    e1.record(stream); torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / n * 1e3
    # x read, y written; + the float32 mask read ('tensor') or the LCSA row / column terms (inline)
    nbytes = B * H * W * (c * 2 + c * 2) + (B * H * W * 9 * 4 if variant == 'tensor' else 4 * (B * H * c + B * W * Cp + W * Cp))
    return {'us': us, 'bytes': nbytes, 'gbs': nbytes / (us * 1e-6) / 1e9, 'shape': [B, H, W, c], 'variant': variant}


def c4_cpu_model():
    import kadcnet
    torch.set_num_threads(os.cpu_count() or 1)
    return kadcnet.load_model(None, 'raw', 'cpu', randomize=True, seed=0)


def c4_cpu_step(model, img):
    """One image through the plain PyTorch modules (what the reference's raw backend executes) + NMS, fp32, all host cores."""
    from kadcnet.postprocess import non_max_suppression
    t0 = time.perf_counter()
    with torch.no_grad():
        non_max_suppression(model(img.float() / 255), C4['conf'], C4['iou'], max_det=C4['max_det'])
    return time.perf_counter() - t0


def c4_cpu_sample(n_images=5, warmup=2):
    """Median over `n_images` single-image steps after `warmup` untimed ones; returns (images/s, n, seconds)."""
    model = c4_cpu_model()
    imgs = c4_images(n_images + warmup)
    for i in range(warmup):
        c4_cpu_step(model, imgs[i:i + 1])
    ts = [c4_cpu_step(model, imgs[warmup + i:warmup + i + 1]) for i in range(n_images)]
    return 1.0 / statistics.median(ts), n_images, sum(ts)


def c4_torch_gpu_sample(device, mb=8, iters=3):
    """The same plain PyTorch modules in fp16 on the GPU (library kernels: cuDNN, torchvision deform_conv2d and nms), eager, the
    way the reference's 'raw' backend runs on a GPU. A secondary yardstick next to the CPU arm; not this package's code path."""
    import kadcnet
    from kadcnet.postprocess import non_max_suppression
    model = kadcnet.load_model(None, 'raw', str(device), randomize=True, seed=0).half()
    imgs = c4_images(mb, seed=7).to(device)

    def once():
        with torch.no_grad():
            return non_max_suppression(model(imgs.half() / 255), C4['conf'], C4['iou'], max_det=C4['max_det'])
    for _ in range(2):
        once()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        once()
    e1.record(); torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    return {'value': mb / (ms * 1e-3), 'unit': 'images/s', 'ms_per_mini_batch': ms, 'mini_batch': mb, 'dtype': 'f16',
            'what': 'plain PyTorch modules + torchvision deform_conv2d + reference-order NMS on the same GPU, eager (library kernels only)'}


def run_c4(args, rank, world, local):
    import kadcnet
    from kadcnet.postprocess import non_max_suppression_device as non_max_suppression
    from kadcnet.runtime import StaticGraph
    from kadcnet.sharding import gather_detections, shard_range
    from kadconv import _abi, ops
    device = torch.device('cuda', local)
    torch.cuda.set_device(device)
    host_group = torch.distributed.new_group(backend='gloo') if world > 1 else None
    fast = kadcnet.load_model(None, 'optimized', str(device), randomize=True, seed=0, dtype=torch.float16, conv3x3=args.conv3x3)
    # the job's images are sharded by batch: rank r owns images [r*64, (r+1)*64) of the step's 64 * world (its share is generated
    # from its own seed, which is what slicing one seeded global batch would amount to)
    a, b = shard_range(C4['images'] * world, rank, world)
    n_local = b - a
    host = c4_images(n_local, seed=rank).pin_memory()
    dev = host.to(device)
    mb = max(1, min(args.mini_batch, n_local))
    while n_local % mb:
        mb -= 1
    stream = torch.cuda.current_stream()

    def forward(u8):
        return fast(u8)[0]        # uint8 in: normalisation and layout change are one kernel of the engine

    forward(dev[:mb])                     # the first forward also packs every layer's weights (one-off launches): not counted
    k0 = _abi.KERNELS_LAUNCHED[0]
    forward(dev[:mb])
    kernels_per_mb = _abi.KERNELS_LAUNCHED[0] - k0
    if args.profile:
        # short eager run for a profiler's launch list: one warm mini-batch, then one forward + NMS under an NVTX-free region
        torch.cuda.synchronize()
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record(); d = non_max_suppression(forward(dev[:mb]), C4['conf'], C4['iou'], max_det=C4['max_det']); t1.record()
        torch.cuda.synchronize()
        return {'metric': 'KAD-CNet-S 800x800 images/s', 'value': mb / (t0.elapsed_time(t1) * 1e-3), 'unit': 'images/s', 'n_gpus': world,
                'config': {'workload': f'c4 profile run: one eager mini-batch of {mb} images'}, 'own_kernels_per_mini_batch': kernels_per_mb,
                'e2e': None, 'gpu_launches': kernels_per_mb}
    graphs = {}

    def run_mb(u8):
        n = u8.shape[0]
        if n not in graphs:
            graphs[n] = StaticGraph(forward, u8)
        y = graphs[n](u8, clone=False)
        return non_max_suppression(y, C4['conf'], C4['iou'], max_det=C4['max_det'])

    # Both timed legs go through the streaming API (kadcnet.pipeline.DetectionPipeline): the forward graph of mini-batch i+1 overlaps
    # the batched NMS of mini-batch i (a second stream), as a serving loop would run it. `value`: the images are resident in HBM;
    # `e2e`: pinned host images in, detections on the host out.
    from kadcnet.pipeline import DetectionPipeline
    # a mini-batch of 64 or more runs as two graphs of half the size side by side (measured: 15.2 ms against 15.6 ms per 64 images;
    # no gain at 32 images and below)
    splits = 2 if (mb >= 64 and mb % 2 == 0) else 1
    pipe = DetectionPipeline(fast, (mb, 3, C4['H'], C4['W']), C4['conf'], C4['iou'], C4['max_det'], device, splits=splits)
    dev_batches = [dev[i:i + mb] for i in range(0, n_local, mb)]
    host_batches = [host[i:i + mb] for i in range(0, n_local, mb)]
    dets = []
    sampler = ClockSampler(local); sampler.start()
    for _ in range(max(args.warmup, 3)):
        dets = [d for batch in pipe.run(dev_batches) for d in batch]
    torch.cuda.synchronize(); ops.check_status(device)
    n_det = sum(t.shape[0] for t in dets)
    barrier(world); torch.cuda.synchronize()
    sampler.begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in pipe.run(dev_batches * args.steps, to_host=False):
        pass
    e1.record(stream)
    torch.cuda.synchronize(); barrier(world)
    clocks = sampler.stop()
    ms_total = max_over_ranks(e0.elapsed_time(e1), world, device)
    # forward-only time of one mini-batch graph (for the roofline line)
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if mb not in graphs:
        graphs[mb] = StaticGraph(forward, dev[:mb])
    graphs[mb](dev[:mb], clone=False)
    g0.record(stream)
    for _ in range(5):
        graphs[mb](dev[:mb], clone=False)
    g1.record(stream); torch.cuda.synchronize()
    fwd_ms = g0.elapsed_time(g1) / 5

    # strong-scaling point of the same sweep: ONE batch of 64 images in total, sharded by batch over the ranks
    # (64 / 32 / 16 / 8 images per GPU at 1 / 2 / 4 / 8 GPUs), same forward graph + NMS per rank, no collective
    sa, sb = shard_range(C4['images'], rank, world)
    n_strong = sb - sa
    if world == 1:
        strong_ms = ms_total / args.steps
    else:
        pipe_s = DetectionPipeline(fast, (n_strong, 3, C4['H'], C4['W']), C4['conf'], C4['iou'], C4['max_det'], device)
        for _ in pipe_s.run([dev[:n_strong]] * 3, to_host=False):
            pass
        barrier(world); torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(stream)
        for _ in pipe_s.run([dev[:n_strong]] * args.steps, to_host=False):
            pass
        s1.record(stream)
        torch.cuda.synchronize(); barrier(world)
        strong_ms = max_over_ranks(s0.elapsed_time(s1), world, device) / args.steps
    strong = {'scaling': 'strong', 'images_total': C4['images'], 'images_per_rank': n_strong, 'value': C4['images'] / (strong_ms * 1e-3),
              'unit': 'images/s', 'ms_per_step': strong_ms}

    # latency of one image (BASELINE configs[3]: batch 1, 800x800): forward graph + NMS, and the same from a pinned host image
    # to detections on the host
    c3 = None
    if rank == 0:
        one = dev[:1]
        for _ in range(3):
            run_mb(one)
        torch.cuda.synchronize()
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_lat = 30
        l0.record(stream)
        for _ in range(n_lat):
            run_mb(one)
        l1.record(stream); torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n_lat):
            d = run_mb(host[:1].to(device, non_blocking=True))
            d = [t.cpu() for t in d]
        host_ms = (time.perf_counter() - t0) / n_lat * 1e3
        c3 = {'workload': 'c3: one uint8 3x800x800 image, fp16, forward graph + NMS (conf 0.001, IoU 0.65)', 'ms_per_image': l0.elapsed_time(l1) / n_lat,
              'e2e_ms_per_image': host_ms, 'detections': int(d[0].shape[0]), 'launches_per_image': kernels_per_mb + 1}

    # end to end: per step the H2D copy of the step's images and the D2H copy of its detections are inside the timed region
    n_e2e = max(2, args.steps)                 # the same K steps as the device-resident leg (the pipeline's fill and drain are inside)
    for _ in pipe.run(host_batches):            # warm-up (graph capture happened in the constructor)
        pass
    torch.cuda.synchronize(); barrier(world)
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    dets_host = []
    for d in pipe.run(host_batches * n_e2e):
        dets_host = d if len(host_batches) == 1 else dets_host + d
    f1.record(stream)
    torch.cuda.synchronize(); barrier(world)
    dets_host = dets_host[-n_local:]
    e2e_ms = max_over_ranks(f0.elapsed_time(f1), world, device) / n_e2e
    ops.check_status(device)
    all_d = gather_detections(dets_host, rank, world, group=host_group)     # final host gather to rank 0
    n_total = sum(t.shape[0] for t in all_d) if rank == 0 else None
    pk = peaks()
    ips_fwd = mb / (fwd_ms * 1e-3)
    dom = c4_dominant_kernel(device, mb, stream)
    return {
        'metric': 'KAD-CNet-S 800x800 images/s', 'value': C4['images'] * world * args.steps / (ms_total * 1e-3), 'unit': 'images/s',
        'n_gpus': world, 'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': ms_total / args.steps,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f16', 'data': 'synthetic',
        'config': {'workload': C4_WORKLOAD, 'l2': C4_L2},
        'run': {'images_per_rank': n_local, 'mini_batch': mb, 'l2': f'activations of a mini-batch of {mb} images exceed the 126 MB L2',
                'detections_per_step_rank0': n_det, 'detections_gathered': n_total, 'forward': ('two CUDA graphs of half a mini-batch replayed side by side on two streams' if splits == 2 else 'CUDA graph per mini-batch shape'),
                'nms': 'one batched CUDA kernel per mini-batch (kad_nms_batched) on a second stream: it overlaps the forward graph of the next mini-batch',
                'conv3x3': 'library (cuDNN through torch) + kad_bias_act' if args.conv3x3 == 'library' else 'kad_conv3x3_bias_act (tcgen05)'},
        'strong_scaling': strong, 'c3_latency': c3,
        'roofline': {'bound': 'hbm', 'achieved': dom['gbs'], 'peak': pk['hbm_gbs'], 'unit': 'GB/s', 'frac': dom['gbs'] / pk['hbm_gbs'],
                     'traffic': NCU_TRAFFIC['c4_dsc_mma'], 'peak_source': pk['_source'],
                     'kernel': 'dsc_mma_kernel (offset convolution + deformable convolution of a KAD-Conv branch), the largest '
                               'share of the forward; timed alone on its largest detector shape', 'shape': dom['shape'],
                     'us_per_launch': dom['us'], 'algorithmic_bytes': dom['bytes'],
                     'limiter': 'shared-memory data pipe', 'lsu_pipe_frac': NCU_LSU_PIPE['c4_dsc_mma'], 'issue_slot_frac': NCU_ISSUE['c4_dsc_mma'],
                     'note': 'HBM is not what limits this kernel (12-channel maps: 84 bytes per pixel against about 2570 warp instructions and about '
                             '1100 shared-memory wavefronts per 32 pixels of bilinear gather): `frac` relates it to the HBM roofline as the contract '
                             'asks; `lsu_pipe_frac` and `issue_slot_frac` are how busy the L1 / shared-memory data pipe and the issue slots are in '
                             'the committed ncu summary (profiles/dsc_mma_kernel_c4.md)'},
        'roofline_forward_graph': {'bound': 'hbm', 'achieved': ips_fwd * C4_MIN_BYTES_PER_IMAGE / 1e9, 'peak': pk['hbm_gbs'], 'unit': 'GB/s',
                                   'frac': ips_fwd * C4_MIN_BYTES_PER_IMAGE / 1e9 / pk['hbm_gbs'],
                                   'kernel': 'whole forward graph (minimum activation traffic 0.35 GB/image, fp16)',
                                   'forward_ms_per_mini_batch': fwd_ms, 'tensor_frac': ips_fwd * C4_GFLOP_PER_IMAGE / 1e3 / pk['bf16_tflops_sustained']},
        'e2e': {'value': C4['images'] * world / (e2e_ms * 1e-3), 'unit': 'images/s', 'h2d_bytes_per_step': host.numel() * world,
                'd2h_bytes_per_step': int(sum(t.numel() * 4 for t in dets_host)) * world, 'ms_per_step': e2e_ms},
        # own kernels of one forward were counted on an eager mini-batch; every one of the `splits` graphs replays them, plus one NMS launch
        'gpu_launches': args.steps * (n_local // mb) * (kernels_per_mb * splits + 1) * world, 'own_kernels_per_mini_batch': kernels_per_mb * splits + 1,
        'clocks': clocks,
    }


# ------------------------------------------------------------------------------------------- C2
C2 = dict(B=16, C=128, H=200, W=200, Cout=256, se_hidden=16)


class OpTimer:
    """Wraps the kadconv.ops entry points with CUDA events so that a composite forward reports per-kernel-group times."""
    NAMES = ['pool_project', 'avg_pool', 'lcsa_mask', 'dsc_forward', 'se_excite', 'merge_upsample_residual', 'se_squeeze', 'se_rescale',
             'gemm1x1_bias_act', 'to_nhwc', 'to_nchw']

    def __init__(self, ops):
        self.ops, self.orig, self.events = ops, {}, []

    def __enter__(self):
        for n in self.NAMES:
            f = getattr(self.ops, n)
            self.orig[n] = f

            def wrapped(*a, _f=f, _n=n, **k):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); r = _f(*a, **k); e1.record()
                self.events.append((_n, e0, e1))
                return r
            setattr(self.ops, n, wrapped)
        return self

    def __exit__(self, *exc):
        for n, f in self.orig.items():
            setattr(self.ops, n, f)

    def totals(self):
        torch.cuda.synchronize()
        out = {}
        for n, e0, e1 in self.events:
            d = out.setdefault(n, [0, 0.0]); d[0] += 1; d[1] += e0.elapsed_time(e1)
        return out


# 3x3 convolutions of KAD-CNet-S at 800x800 (Cin, Cout, stride, input size); the model runs each at batch = mini-batch
CONV3X3_SHAPES = [(144, 144, 1, 100), (64, 64, 1, 100), (96, 96, 1, 50), (40, 72, 2, 400), (72, 144, 2, 199), (144, 64, 1, 100), (32, 32, 1, 200),
                  (216, 144, 1, 50), (144, 216, 2, 99), (144, 144, 1, 50), (128, 128, 1, 25), (144, 112, 2, 99), (216, 288, 2, 49), (216, 64, 1, 50),
                  (288, 144, 1, 25), (216, 144, 2, 49), (144, 144, 1, 25), (288, 64, 1, 25)]


def run_conv3x3(args, local):
    """The detector's 3x3 convolution shapes (+ bias + SiLU, fp16, batch = --mini-batch): this package's tcgen05 kernel next to
    the library path the engine uses by default (cuDNN convolution + kad_bias_act). --profile: the first shape only, own kernel only."""
    import torch.nn.functional as F
    from kadconv import ops
    device = torch.device('cuda', local); torch.cuda.set_device(device)
    B, dt = args.mini_batch, torch.float16
    rows, tot = [], [0.0, 0.0]
    g = torch.Generator(device='cpu').manual_seed(0)
    for cin, cout, s, H in (CONV3X3_SHAPES[:1] if args.profile else CONV3X3_SHAPES):
        x = torch.randn((B, H, H, cin), generator=g).to(device, dt)
        w = (torch.randn((cout, cin, 3, 3), generator=g) / (9 * cin) ** 0.5).to(device, dt)
        b = torch.randn((cout,), generator=g).to(device)
        wp = ops.pack_conv3x3_weight(w, dt).to(device)
        wl = w.contiguous(memory_format=torch.channels_last)

        def own():
            return ops.conv3x3_bias_act(x, wp, b, stride=s)

        def lib():
            return ops.bias_act_(F.conv2d(x.permute(0, 3, 1, 2), wl, None, s, 1).permute(0, 2, 3, 1), b, ops.ACT_SILU)
        us = []
        for fn in ((own,) if args.profile else (own, lib)):
            for _ in range(max(3, args.warmup)):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n = max(2, min(args.steps, 20))
            e0.record()
            for _ in range(n):
                fn()
            e1.record(); torch.cuda.synchronize()
            us.append(1e3 * e0.elapsed_time(e1) / n)
        Ho = (H - 1) // s + 1
        flops = 2.0 * 9 * cin * cout * B * Ho * Ho
        row = {'shape': f'{cin}->{cout} s{s} @{H}', 'own_us': round(us[0], 1), 'own_tflops': round(flops / us[0] / 1e6, 1)}
        tot[0] += us[0]
        if len(us) > 1:
            row.update({'library_us': round(us[1], 1), 'library_tflops': round(flops / us[1] / 1e6, 1)})
            tot[1] += us[1]
        rows.append(row)
    ops.check_status(device)
    return {'metric': 'KAD-CNet-S 3x3 convolutions + bias + SiLU, us per launch', 'unit': 'us', 'batch': B, 'dtype': 'f16',
            'total_own_us': round(tot[0], 1), 'total_library_us': round(tot[1], 1) if tot[1] else None, 'shapes': rows}


# fused 1x1 convolutions (Conv k=1 + folded BN + SiLU) of KAD-CNet-S at 800x800: (Cin, Cout, map size)
GEMM1X1_SHAPES = [(72, 64, 200), (128, 72, 200), (144, 128, 100), (64, 32, 100), (64, 64, 100), (256, 144, 100), (360, 128, 100), (216, 192, 50),
                  (96, 48, 50), (96, 96, 50), (384, 216, 50), (504, 192, 50), (328, 192, 50), (288, 256, 25), (128, 64, 25), (128, 128, 25),
                  (512, 288, 25), (288, 128, 25), (432, 256, 25)]


def run_gemm1x1(args, local):
    """The detector's 1x1 GEMM + bias + SiLU shapes (fp16, batch = --mini-batch) on gemm1x1_tc_kernel: microseconds and achieved
    GB/s of the algorithmic bytes 2*M*(K+N) + 2*K*N against the measured HBM peak. --profile: the (256, 144, 100) shape only, or the one given by --gemm-shape."""
    from kadconv import ops
    device = torch.device('cuda', local); torch.cuda.set_device(device)
    B, dt = args.mini_batch, torch.float16
    peak = peaks(); src = peak['_source']
    rows, tot, tot_floor = [], 0.0, 0.0
    g = torch.Generator(device='cpu').manual_seed(0)
    one = tuple(int(v) for v in args.gemm_shape.split(',')) if args.gemm_shape else (256, 144, 100)
    for K, N, H in ([one] if (args.profile or args.gemm_shape) else GEMM1X1_SHAPES):
        x = torch.randn((B, H, H, K), generator=g).to(device, dt)
        w = (torch.randn((N, K), generator=g) / K ** 0.5).to(device, dt)
        b = torch.randn((N,), generator=g).to(device)
        for _ in range(max(3, args.warmup)):
            ops.gemm1x1_bias_act(x, w, b, act=ops.ACT_SILU)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = max(2, min(args.steps, 20))
        e0.record()
        for _ in range(n):
            ops.gemm1x1_bias_act(x, w, b, act=ops.ACT_SILU)
        e1.record(); torch.cuda.synchronize()
        us = 1e3 * e0.elapsed_time(e1) / n
        M = B * H * H
        nbytes = 2.0 * M * (K + N) + 2.0 * K * N
        gbs = nbytes / us / 1e3
        rows.append({'shape': f'{K}->{N} @{H}', 'us': round(us, 1), 'gb_per_s': round(gbs), 'hbm_frac': round(gbs / peak['hbm_gbs'], 3),
                     'tflops': round(2.0 * M * K * N / us / 1e6, 1)})
        tot += us; tot_floor += nbytes / peak['hbm_gbs'] / 1e3
    ops.check_status(device)
    return {'metric': 'KAD-CNet-S 1x1 GEMM + bias + SiLU, us per launch', 'unit': 'us', 'batch': B, 'dtype': 'f16', 'total_us': round(tot, 1),
            'hbm_floor_us': round(tot_floor, 1), 'peak_gb_per_s': peak['hbm_gbs'], 'peak_source': src, 'shapes': rows}


def run_c2(args, rank, world, local):
    import kadconv
    import kadconv.fast as fast
    from kadconv import _abi, ops
    device = torch.device('cuda', local)
    torch.cuda.set_device(device)
    dt, s = torch.bfloat16, 2
    B, C, H, W, Co, Hd = C2['B'], C2['C'], C2['H'], C2['W'], C2['Cout'], C2['se_hidden']
    g = torch.Generator().manual_seed(0)
    layer = kadconv.KADConv(C).eval()
    with torch.no_grad():
        for name, m in layer.named_modules():
            if isinstance(m, torch.nn.BatchNorm2d):
                m.running_mean.normal_(0, 0.1, generator=g); m.running_var.uniform_(0.5, 1.5, generator=g)
                m.weight.uniform_(0.5, 1.5, generator=g); m.bias.normal_(0, 0.1, generator=g)
            elif name.endswith('conv_offset'):
                m.weight.normal_(0, 0.5 / m.weight[0].numel() ** 0.5, generator=g); m.bias.normal_(0, 0.05, generator=g)
        for w in layer.weight:
            w[0].weight.normal_(0, 1, generator=g)                 # branch scales ~ N(0,1)
    layer = kadconv.enable_fast_inference(layer.to(device))
    w11h = (torch.randn((Co, C), generator=g) / C ** 0.5).to(device, dt); b11 = (0.1 * torch.randn(Co, generator=g)).to(device)
    se = [t.to(device) for t in (torch.randn((Hd, Co), generator=g) / Co ** 0.5, 0.1 * torch.randn(Hd, generator=g),
                                 torch.randn((Co, Hd), generator=g) / Hd ** 0.5, 0.1 * torch.randn(Co, generator=g))]
    xs = [torch.randn((B, H, W, C), generator=g).to(device, dt) for _ in range(2)]     # NHWC, 164 MB each

    def step(i):
        y = fast.kadconv_forward_nhwc(layer, xs[i & 1])
        z = ops.gemm1x1_bias_act(ops.avg_pool(y, 2), w11h, b11, act=ops.ACT_SILU)        # stride-2 pool, then 1x1 GEMM + bias + SiLU on tcgen05
        att = ops.se_excite(ops.se_squeeze(z), (H // 2) * (W // 2), *se)
        return ops.se_rescale(z, att)

    sampler = ClockSampler(local); sampler.start()
    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize(); ops.check_status(device)
    k0 = _abi.KERNELS_LAUNCHED[0]
    barrier(world); torch.cuda.synchronize()
    sampler.begin()
    stream = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    torch.cuda.synchronize(); barrier(world)
    clocks = sampler.stop()
    launches = _abi.KERNELS_LAUNCHED[0] - k0
    ms_total = max_over_ranks(e0.elapsed_time(e1), world, device)
    if args.profile:
        return {'metric': 'KAD-Conv downsampling composition (bf16) feature maps/s', 'value': world * B * args.steps / (ms_total * 1e-3),
                'unit': 'images/s', 'n_gpus': world, 'config': {'workload': 'c2 profile run'}, 'e2e': None, 'gpu_launches': launches}
    with OpTimer(ops) as tm:
        for i in range(4):
            step(i)
    tot = tm.totals()
    pk = peaks()
    px = B * H * W
    widths = [C - (C // 3) * 2, C // 3, C // 3]
    alg = {   # algorithmic bytes per step of each kernel group: inputs read once + outputs written once, s bytes per element
        'pool_project': sum(s * (px * C + (px >> (2 * i)) * c) for i, c in enumerate(widths)),
        'avg_pool': s * (px * C + (px // 4) * C), 'gemm1x1_bias_act': s * ((px // 4) * (C + Co) + C * Co),
        'lcsa_mask': sum((px >> (2 * i)) * (s * c + 4 * 9) for i, c in enumerate(widths)),
        'dsc_forward': sum((px >> (2 * i)) * (s * (c + c) + 4 * 27) + (px >> (2 * i)) * (s * c + 4 * 18) for i, c in enumerate(widths)),
        'merge_upsample_residual': 2 * s * px * C + sum(s * (px >> (2 * i)) * c for i, c in enumerate(widths)),
        'se_squeeze': s * (px // 4) * Co, 'se_rescale': 2 * s * (px // 4) * Co, 'se_excite': 0,
    }
    stages = []
    for n, (cnt, ms) in sorted(tot.items(), key=lambda kv: -kv[1][1]):
        us = ms * 1e3 / 4
        gbs = alg.get(n, 0) / (us * 1e-6) / 1e9 if us > 0 else 0.0
        stages.append({'op': n, 'calls_per_step': cnt // 4, 'us_per_step': us, 'algorithmic_MB': alg.get(n, 0) / 1e6, 'GB_per_s': gbs,
                       'frac_of_hbm_peak': gbs / pk['hbm_gbs']})
    top = stages[0]
    return {
        'metric': 'KAD-Conv downsampling composition (bf16) feature maps/s', 'value': world * B * args.steps / (ms_total * 1e-3), 'unit': 'images/s',
        'n_gpus': world, 'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': ms_total / args.steps, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
        'config': {'workload': 'c2: x[16,128,200,200] bf16 -> KADConv(128) (branch scales N(0,1)) -> avg-pool 2 -> 1x1 GEMM 128->256 + bias + SiLU (tcgen05) -> SE (hidden 16) '
                               '-> rescale; a composition of reference classes (no such module exists in the reference)',
                   'l2': 'two 164 MB inputs alternated', 'layout': 'NHWC'},
        'roofline': {'bound': 'hbm', 'achieved': top['GB_per_s'], 'peak': pk['hbm_gbs'], 'unit': 'GB/s', 'frac': top['frac_of_hbm_peak'],
                     'traffic': None, 'kernel': top['op'], 'peak_source': pk['_source']},
        'stages': stages, 'e2e': None, 'gpu_launches': launches, 'clocks': clocks,
    }

# ------------------------------------------------------------------------------------------- C0
def run_c0(args, local):
    """BASELINE configs[0]: KADConv(64) on x[2,64,80,80] fp32 (the reference's CPU-runnable case). Microseconds per forward of the
    module with the B200 pipeline enabled (NCHW in, NCHW out, eager launches), of the plain PyTorch module on the same GPU, and of
    the plain module on the host cores."""
    import kadconv
    device = torch.device('cuda', local); torch.cuda.set_device(device)
    torch.manual_seed(0)
    layer = kadconv.KADConv(64).eval()
    g = torch.Generator().manual_seed(0)
    with torch.no_grad():
        for name, m in layer.named_modules():
            if name.endswith('conv_offset'):      # the reference zero-initialises it: give the offsets a spread of about 0.5 px
                m.weight.normal_(0, 0.5 / m.weight[0].numel() ** 0.5, generator=g); m.bias.normal_(0, 0.05, generator=g)
    x = torch.randn((2, 64, 80, 80), generator=g)

    def timed(fn, n):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n * 1e3

    n = max(10, args.steps)
    xd = x.to(device)
    plain = layer.to(device)
    with torch.no_grad():
        ref = plain(xd)
        us_torch = timed(lambda: plain(xd), n)
        kadconv.enable_fast_inference(plain)
        y = plain(xd)
        us_ours = timed(lambda: plain(xd), n)
    err = (y - ref).abs().max().item()
    kadconv.disable_fast_inference(plain)
    cpu = plain.cpu()
    torch.set_num_threads(os.cpu_count() or 1)
    with torch.no_grad():
        cpu(x)
        t0 = time.perf_counter()
        for _ in range(5):
            cpu(x)
        us_cpu = (time.perf_counter() - t0) / 5 * 1e6
    model, cores = cpu_info()
    return {'metric': 'KAD-Conv op (KADConv(64), x[2,64,80,80] fp32) forwards/s', 'value': 1e6 / us_ours, 'unit': 'forwards/s', 'n_gpus': 1,
            'steps': n, 'warmup': 5, 'ms_per_step': us_ours / 1e3, 'us_per_forward': us_ours, 'higher_is_better': True, 'vs_baseline': None,
            'dtype': 'f32', 'data': 'synthetic', 'config': {'workload': 'c0: KADConv(64), x[2,64,80,80] fp32, module API (NCHW in / out), eager'},
            'max_abs_vs_plain_module_on_gpu': err,
            'torch_gpu_reference': {'us_per_forward': us_torch, 'what': 'the plain PyTorch module on the same GPU (torchvision deform_conv2d)'},
            'cpu_baseline': {'value': 1e6 / us_cpu, 'unit': 'forwards/s', 'us_per_forward': us_cpu, 'cores': torch.get_num_threads(), 'kind': 'port',
                             'sample': '5 forwards of the plain module, fp32', 'cpu': model, 'os_cpu_count': cores},
            'e2e': None, 'gpu_launches': n * 27}


# ------------------------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default='c4', choices=['c0', 'c1', 'c2', 'c4', 'c4-kernel', 'conv3x3', 'gemm1x1'],
                    help='c4 (default): KAD-CNet-S images/s, with the KAD-Conv op of c1 timed in the same run; c1 / c2: the operator configurations alone')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--mini-batch', type=int, default=64, help='c4: images per forward graph')
    ap.add_argument('--conv3x3', default='library', choices=['library', 'tcgen05'],
                    help="c4: 3x3 convolutions through the library (default, faster at this model's widths) or this package's tcgen05 kernel")
    ap.add_argument('--profile', action='store_true', help='short run for ncu: no e2e leg, no CPU baseline')
    ap.add_argument('--gemm-shape', default=None, help="gemm1x1: one shape 'Cin,Cout,map' instead of the detector's 19")
    args = ap.parse_args()
    # stdout carries exactly one JSON line: anything libraries print while they initialise (NCCL's version banner) goes to stderr
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(obj), flush=True)
        os.dup2(2, 1)

    if args.impl == 'reference':
        # the reference's plain PyTorch path on the host cores. No process group is created: under torchrun rank 0 alone
        # works, the other ranks leave at once. One step = one unit of the workload (one image / one feature map); the
        # line reports the steps it really ran and the measured time of one step.
        rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
        if rank != 0:
            return
        model_name, cores = cpu_info()
        steps, warm = max(1, args.steps), max(0, args.warmup)
        if args.workload == 'c4':
            model = c4_cpu_model()
            imgs = c4_images(min(steps + warm, 16))
            for i in range(warm):
                c4_cpu_step(model, imgs[i % len(imgs):i % len(imgs) + 1])
            t0 = time.perf_counter()
            ts = [c4_cpu_step(model, imgs[(warm + i) % len(imgs):(warm + i) % len(imgs) + 1]) for i in range(steps)]
            total = time.perf_counter() - t0
            metric, workload, unit_name = 'KAD-CNet-S 800x800 images/s', C4_WORKLOAD, 'image 3x800x800'
            what = 'fp32 plain PyTorch modules (the op sequence of the reference\'s raw backend) + torchvision deform_conv2d + NMS'
        else:
            t = c1_cpu_inputs()
            for i in range(warm):
                c1_cpu_step(*t, i % C1['B'])
            t0 = time.perf_counter()
            ts = [c1_cpu_step(*t, (warm + i) % C1['B']) for i in range(steps)]
            total = time.perf_counter() - t0
            metric, workload, unit_name = 'KAD-Conv op (DSC 256->256 @100x100 fp16) feature maps/s', C1_WORKLOAD, 'feature map [1,256,100,100]'
            what = 'fp32 torchvision.ops.deform_conv2d (the call DSC.forward makes)'
        v = steps / total
        emit({
            'impl': 'reference', 'metric': metric, 'value': v, 'unit': 'images/s', 'n_gpus': world, 'steps': steps, 'warmup': warm,
            'ms_per_step': 1e3 * total / steps, 'ms_per_step_median': 1e3 * statistics.median(ts), 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic', 'config': {'workload': workload, 'l2': C4_L2 if workload == C4_WORKLOAD else C1_L2},
            'run': {'step': f'one {unit_name} of the workload per step (a bounded sample: the host cores need about {64 * total / steps:.0f} s for '
                            'the 64 images of one GPU step)' if args.workload == 'c4' else f'one {unit_name} of the batch of 16 per step'},
            'cpu_baseline': {'value': v, 'unit': 'images/s', 'cores': torch.get_num_threads(), 'kind': 'port',
                             'sample': f'{steps} steps of one {unit_name} after {warm} warm-up steps, {what}', 'cpu': model_name, 'os_cpu_count': cores},
            'e2e': {'value': v, 'unit': 'images/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}})
        return

    rank, world, local = dist_setup(args.gpus)

    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device (the product has no CPU path); use --impl reference for the CPU baseline')
    if args.workload == 'c4-kernel':
        # the detector's dominant kernel alone (what the `roofline` object of the c4 line is measured on); small enough for ncu
        device = torch.device('cuda', local); torch.cuda.set_device(device)
        dom = c4_dominant_kernel(device, args.mini_batch, torch.cuda.current_stream(), n=max(3, min(args.steps, 20)))
        old = None if args.profile else c4_dominant_kernel(device, args.mini_batch, torch.cuda.current_stream(), n=max(3, min(args.steps, 20)), variant='inline')
        if rank == 0:
            emit(({'metric': 'dsc_mma_kernel us per launch', 'value': dom['us'], 'unit': 'us', 'shape': dom['shape'],
                   'algorithmic_bytes': dom['bytes'], 'gb_per_s': dom['gbs'], 'gpu_launches': max(3, min(args.steps, 20)),
                   'inline_mask_variant_us': old['us'] if old else None}))
        return
    if args.workload in ('conv3x3', 'gemm1x1', 'c0'):
        res = run_conv3x3(args, local) if args.workload == 'conv3x3' else (run_gemm1x1(args, local) if args.workload == 'gemm1x1' else run_c0(args, local))
        if rank == 0:
            emit(res)
        return
    res = {'c1': run_c1, 'c2': run_c2, 'c4': run_c4}[args.workload](args, rank, world, local)
    if args.workload == 'c4' and not args.profile:
        # the second half of the metric: the KAD-Conv operator alone (c1), timed in the same run
        import copy
        a1 = copy.copy(args); a1.steps = 20; a1.warmup = 3; a1.profile = True
        op = run_c1(a1, rank, world, local)
        res['kadconv_op'] = {'workload': op['config']['workload'], 'us_per_op': op['us_per_op'], 'feature_maps_per_s': op['value'],
                             'roofline': op['roofline']}
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline and not args.profile and args.workload in ('c1', 'c4'):
            model, cores = cpu_info()
            device = torch.device('cuda', local)
            if args.workload == 'c4':
                ips, n, dt = c4_cpu_sample()
                sample = f'median of {n} single-image steps ({dt:.1f} s), fp32 plain PyTorch modules + torchvision deform_conv2d + NMS'
                try:
                    res['torch_gpu_reference'] = c4_torch_gpu_sample(device)
                    res['kadconv_op']['torch_gpu_reference'] = c1_torch_gpu_sample(device)
                except Exception as e:      # the library op may be missing for this GPU: say so instead of failing the line
                    res['torch_gpu_reference'] = {'unavailable': f'{type(e).__name__}: {e}'[:300]}
            else:
                ips, n, dt = c1_cpu_sample()
                sample = f'median of {n} single-map steps of the 16 c1 feature maps ({dt:.1f} s), fp32, torchvision.ops.deform_conv2d (the call DSC.forward makes)'
                try:
                    res['torch_gpu_reference'] = c1_torch_gpu_sample(device)
                except Exception as e:
                    res['torch_gpu_reference'] = {'unavailable': f'{type(e).__name__}: {e}'[:300]}
            res['cpu_baseline'] = {'value': ips, 'unit': 'images/s', 'cores': torch.get_num_threads(), 'kind': 'port', 'sample': sample,
                                   'cpu': model, 'os_cpu_count': cores}
        emit(res)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
