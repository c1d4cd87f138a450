#!/usr/bin/env python
"""Benchmark of the KAD-Conv inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c4] [--impl ours|reference]

Prints ONE JSON line (rank 0). Workloads (BASELINE.json configs):
  c1  KAD-Conv operator: DSC 256->256, [16,256,100,100] fp16, offsets N(0,2) px, mask given
      (gather + tcgen05 implicit GEMM). One step = one pass over the batch of 16 feature maps.
  c4  KAD-CNet-S detector, fp16, 3x800x800 synthetic images, batch 64 sharded over the ranks,
      backbone + neck + head + NMS. One step = one pass over the 64 images.
`value` is whole-job images/s with inputs resident in HBM; `e2e` is the same metric through the
public Python API with pinned-host inputs and a host read of the result inside the timed region.
`--impl reference` times the CPU oracle port (plain PyTorch + torchvision on the host cores) on a
bounded sample of the same workload.
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
NCU_TRAFFIC = {'c1': None}   # DRAM bytes per launch from the committed ncu summary (profiles/), filled below
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
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.index), f'--query-gpu={self.Q}', '--format=csv,noheader,nounits',
                                          '-lms', '100'], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for ln in self.lines:
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
        dist.init_process_group(backend)
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


def c1_cpu_sample(seconds_target=12.0, max_images=16):
    """torchvision.ops.deform_conv2d (what DSC.forward calls in the reference) in fp32 on all host cores."""
    import torchvision
    torch.set_num_threads(os.cpu_count() or 1)
    x, off, msk, w, b = c1_inputs('cpu', 0)
    x, off, msk, w = x.float(), off.float(), msk.float(), w.float()
    with torch.no_grad():
        torchvision.ops.deform_conv2d(x[:1], off[:1], w, b, stride=1, padding=1, mask=msk[:1])   # warm-up
        t0 = time.perf_counter(); n = 0
        while n < max_images and (time.perf_counter() - t0) < seconds_target:
            torchvision.ops.deform_conv2d(x[n:n + 1], off[n:n + 1], w, b, stride=1, padding=1, mask=msk[n:n + 1])
            n += 1
        dt = time.perf_counter() - t0
    return n / dt, n, dt


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

    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize(); ops.check_status(device)
    sampler = ClockSampler(local); sampler.start()
    barrier(world); torch.cuda.synchronize()
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

    for i in range(2):
        e2e_step(i)
    torch.cuda.synchronize(); barrier(world)
    n_e2e = max(2, min(args.steps, 10))
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    for i in range(n_e2e):
        e2e_step(i)
    f1.record(stream)
    torch.cuda.synchronize(); barrier(world)
    e2e_ms = max_over_ranks(f0.elapsed_time(f1), world, device) / n_e2e
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
        'config': {'workload': 'c1: DSC 256->256, x[16,256,100,100] fp16, offsets N(0,2) px, mask sigmoid(N(0,1)), W U(+-1/48)',
                   'per_gpu_batch': C1['B'], 'l2': 'two 174 MB input sets alternated (each larger than the 126 MB L2)',
                   'layout': 'NHWC in HBM'},
        'roofline': {'bound': 'tensor', 'achieved': achieved, 'peak': pk['bf16_tflops'], 'unit': 'TFLOP/s',
                     'frac': achieved / pk['bf16_tflops'], 'traffic': NCU_TRAFFIC['c1'], 'peak_source': pk['_source'] + ' (burst)',
                     'kernel': 'dsc_tc_kernel', 'flops_per_launch': C1_FLOPS, 'algorithmic_bytes': C1_BYTES,
                     'hbm_frac_of_peak': C1_BYTES / (kern_ms * 1e-3) / 1e9 / pk['hbm_gbs']},
        'e2e': {'value': world * C1['B'] / (e2e_ms * 1e-3), 'unit': 'images/s', 'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h,
                'ms_per_step': e2e_ms},
        'gpu_launches': args.steps * 1,
        'clocks': clocks,
    }
    return res


# ------------------------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default='c1', choices=['c1'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    args = ap.parse_args()
    rank, world, local = dist_setup(args.gpus)

    if args.impl == 'reference':
        if rank == 0:
            model, cores = cpu_info()
            vals = []
            for _ in range(max(1, min(args.steps, 3))):
                ips, n, dt = c1_cpu_sample(seconds_target=8.0, max_images=4)
                vals.append(ips)
            v = statistics.median(vals)
            sample = f'{n} feature maps [1,256,100,100] of the c1 batch per step, fp32, torchvision.ops.deform_conv2d'
            print(json.dumps({
                'impl': 'reference', 'metric': 'KAD-Conv op (DSC 256->256 @100x100 fp16) feature maps/s', 'value': v, 'unit': 'images/s',
                'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': 1e3 * C1['B'] / v, 'higher_is_better': True,
                'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
                'config': {'workload': 'c1: DSC 256->256, x[16,256,100,100], offsets N(0,2) px (CPU oracle port, fp32)'},
                'cpu_baseline': {'value': v, 'unit': 'images/s', 'cores': torch.get_num_threads(), 'kind': 'port', 'sample': sample,
                                 'cpu': model, 'os_cpu_count': cores},
                'e2e': {'value': v, 'unit': 'images/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}}))
        return

    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device (the product has no CPU path); use --impl reference for the CPU baseline')
    res = run_c1(args, rank, world, local)
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            model, cores = cpu_info()
            ips, n, dt = c1_cpu_sample()
            res['cpu_baseline'] = {'value': ips, 'unit': 'images/s', 'cores': torch.get_num_threads(), 'kind': 'port',
                                   'sample': f'{n} of the 16 c1 feature maps in {dt:.1f} s, fp32, torchvision.ops.deform_conv2d (the call DSC.forward makes)',
                                   'cpu': model, 'os_cpu_count': cores}
        print(json.dumps(res))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
