"""Benchmark of the Mega-MoE hot path: `python bench.py --gpus N --steps K --warmup W [--impl reference]`.

Metric (BASELINE.json): MoE layer tokens/s (whole job) with the fraction of the B200 roofline that explains it.
One "step" = one pass of the layer over one batch of synthetic tokens:
    router (sigmoid, top-8, renormalise) -> BF16->FP8 per-32 quantisation -> dispatch -> L1 GEMM + SwiGLU + FP8 requant
    -> L2 GEMM -> weighted top-k combine.
N = 1 runs BASELINE config 3 (4096 tokens, hidden 7168, 256 MXFP4 experts, top-8, intermediate 2048).
Prints ONE JSON line (rank 0). `value` is timed with inputs resident in HBM; `e2e` includes the per-step
host->device copy of the inputs (pinned memory) and the device->host copy of y.
`--impl reference` times the CPU restatement of the reference arithmetic (oracle/) on the host cores instead.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CONFIG3 = dict(tokens=4096, hidden=7168, inter=2048, experts=256, topk=8)
METRIC = 'mega_moe_layer_tokens_per_s'
CPU_SAMPLE_EXPERTS = 16  # experts whose routed rows the CPU legs evaluate per pass (both legs time the same rows)
INPUT_SEED = 1234        # CPU generator seed of rank 0's tokens and router logits (rank r uses INPUT_SEED + r)
FP4_DENSE_PEAK_TFLOPS_NOMINAL = 9000.0
FP8_DENSE_PEAK_TFLOPS_NOMINAL = 4500.0
# DRAM bytes (read + write) per algorithmic byte of the gate/up GEMM: dram__bytes_read.sum + dram__bytes_write.sum of
# an ncu capture of the same kernels on a 32-expert, 512-token layer (same rows per expert as the headline workload),
# divided by that case's algorithmic bytes. Traffic grows in proportion to experts and rows, so a full launch is
# this ratio times its own algorithmic bytes.
L1_KERNEL_DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.06
L1_TRAFFIC_SOURCE = 'ncu capture of a 32-expert, 512-token layer (about 128 rows per expert), scaled by algorithmic bytes'


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--tokens', type=int, default=0, help='override tokens per rank (profiling small cases only)')
    ap.add_argument('--experts', type=int, default=0, help='override the expert count (profiling small cases only)')
    ap.add_argument('--skip-cpu-baseline', action='store_true')
    ap.add_argument('--guest-experts', type=int, default=4,
                    help='expert-parallel runs: guest expert slots per rank for the hot-expert row spill (0 = every expert\'s '
                         'rows stay on its owner)')
    ap.add_argument('--comm-sms', type=int, default=-1,
                    help='expert-parallel runs: SMs kept for the kernels that move rows while the GEMMs run (the library\'s '
                         '"ep_comm_sms" knob; -1 = its default, 0 = one stream without overlap)')
    ap.add_argument('--fused-dispatch', type=int, default=-1,
                    help='expert-parallel runs: the library\'s "fused_dispatch" knob (-1 = its default)')
    ap.add_argument('--fused-return', type=int, default=-1,
                    help='expert-parallel runs: the library\'s "fused_return" knob (-1 = its default)')
    ap.add_argument('--pdl', type=int, default=-1, help='programmatic dependent launch: 0 / 1 (-1 = the library\'s default)')
    ap.add_argument('--no-stage-events', action='store_true',
                    help='profiling aid: the timed steps record no CUDA events at the stage boundaries (stages_ms and the '
                         'roofline then come out empty)')
    ap.add_argument('--skip-other-configs', action='store_true',
                    help='N = 1 only: leave out the extra timings (8192-token base, BASELINE configs 1, 2 and 4) after the headline line')
    ap.add_argument('--mma', default='fp8xfp4', choices=['fp8xfp4', 'nvfp4xnvfp4'],
                    help='nvfp4xnvfp4 runs the NVFP4 prefill variant (16384 tokens) instead of the headline workload')
    ap.add_argument('--workload', default='layer', choices=['layer', 'gemm_contiguous', 'gemm_masked', 'bf16_gemm_contiguous', 'bf16_gemm_masked',
                                                            'bf16_gemm_dense', 'bf16_layer', 'k_grouped_gemm'],
                    help='gemm_contiguous / gemm_masked time the stand-alone grouped GEMMs of BASELINE configs 1 and 2 '
                         '(one GPU, not the headline line)')
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d['hbm_gbs']), 'measured'
    return 6650.0, 'fallback'


class NvmlClockSampler:
    """SM clock and throttle reasons of one GPU read through NVML (read-only queries) every few milliseconds by a thread
    of this process, between begin() and end(). Preferred over a nvidia-smi child process, which needs up to a second to
    start and then answers slowly while eight ranks query it at once."""
    REASONS = ((0x8, 'hw_slowdown'), (0x40, 'hw_thermal_slowdown'), (0x20, 'sw_thermal_slowdown'), (0x4, 'sw_power_cap'))

    def __init__(self, gpu_index: int):
        import threading
        import pynvml
        import torch
        self.nvml = pynvml
        pynvml.nvmlInit()
        try:
            self.handle = pynvml.nvmlDeviceGetHandleByUUID(f'GPU-{torch.cuda.get_device_properties(gpu_index).uuid}')
        except Exception:
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        self.max_clock = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        self.query()  # fails here, not in the thread, if a query is unsupported
        self.samples, self.active, self.done = [], False, False
        self.thread = threading.Thread(target=self.run, daemon=True)

    def query(self):
        reasons = getattr(self.nvml, 'nvmlDeviceGetCurrentClocksEventReasons',
                          getattr(self.nvml, 'nvmlDeviceGetCurrentClocksThrottleReasons', None))(self.handle)
        return float(self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM)), int(reasons)

    def run(self):
        while not self.done:
            if self.active:
                try:
                    self.samples.append(self.query())
                except Exception:
                    pass
            time.sleep(0.004)

    def start(self):
        self.thread.start()

    def begin(self):
        self.active = True

    def end(self):
        self.active = False

    def stop(self):
        self.active = False
        if not self.samples:
            self.samples.append(self.query())
        self.done = True
        self.thread.join()
        clocks = sorted(c for c, _ in self.samples)
        mask = 0
        for _, r in self.samples:
            mask |= r
        return {'sm_mhz': clocks[len(clocks) // 2] if clocks else None, 'sm_max_mhz': self.max_clock, 'samples': len(clocks),
                'reasons': sorted(name for bit, name in self.REASONS if mask & bit), 'window': 'timed region', 'source': 'nvml'}


def make_clock_sampler(gpu_index: int):
    try:
        return NvmlClockSampler(gpu_index)
    except Exception:
        return ClockSampler(gpu_index)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (used when NVML cannot be
    loaded in-process). nvidia-smi needs up to a
    second to start on a box with eight GPUs, so it is started before the warm-up and the samples are cut to the timed
    region afterwards by their timestamps (begin() / end() mark it)."""
    FIELDS = ('timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
              'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
              'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.file = tempfile.NamedTemporaryFile('w+', suffix='.csv', delete=False)
        self.proc = None
        self.t_begin = self.t_end = None

    def start(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--query-gpu={self.FIELDS}', '--format=csv,noheader,nounits',
                                          '-lms', '20', '-i', str(self.gpu_index)], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def begin(self):
        import datetime
        self.t_begin = datetime.datetime.now()

    def end(self):
        import datetime
        self.t_end = datetime.datetime.now()

    def stop(self):
        import datetime
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        if self.t_end is None:
            self.end()
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        self.file.flush()
        self.file.seek(0)
        rows = []  # (time, sm clock, max sm clock, reasons)
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 10:
                continue
            try:
                try:
                    when = datetime.datetime.strptime(parts[0], '%Y/%m/%d %H:%M:%S.%f')
                except ValueError:
                    when = None  # unknown timestamp format: keep the sample, it cannot be cut to the window
                rows.append((when, float(parts[2]), float(parts[3]),
                             [name for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'),
                                                        parts[6:10]) if val.lower().startswith('active')]))
            except ValueError:
                continue
        self.file.close()
        os.unlink(self.file.name)
        window = 'timed region'
        if self.t_begin is not None and rows and all(r[0] is not None for r in rows):
            pad = datetime.timedelta(milliseconds=10)
            inside = [r for r in rows if self.t_begin - pad <= r[0] <= self.t_end + pad]
            if not inside and rows:  # a timed region shorter than the sampling period: the samples next to it
                middle = self.t_begin + (self.t_end - self.t_begin) / 2
                inside = sorted(rows, key=lambda r: abs((r[0] - middle).total_seconds()))[:3]
                window = 'nearest samples (timed region shorter than the sampling period)'
            rows = inside
        clocks = sorted(r[1] for r in rows)
        reasons = sorted({name for r in rows for name in r[3]})
        return {'sm_mhz': clocks[len(clocks) // 2] if clocks else None, 'sm_max_mhz': rows[-1][2] if rows else None,
                'samples': len(clocks), 'reasons': reasons, 'window': window}


def cpu_sample_pass(sample):
    """One pass of the oracle over the sampled experts: dequantise weights on the fly, L1, SwiGLU + requant, L2.
    Returns the number of routed rows processed."""
    import torch
    from oracle import moe as omoe
    from oracle import quant
    rows = 0
    for e in range(len(sample['l1_q'])):
        x_q, x_sf, w = sample['x_q'][e], sample['x_sf'][e], sample['w'][e]
        if x_q.shape[0] == 0:
            continue
        acc1 = quant.dequantize_fp8(x_q, x_sf, 32) @ quant.dequantize_fp4(sample['l1_q'][e], sample['l1_sf'][e], 32).T
        a2_q, a2_sf = omoe.swiglu_requant(acc1, w, None)
        acc2 = quant.dequantize_fp8(a2_q, a2_sf, 32) @ quant.dequantize_fp4(sample['l2_q'][e], sample['l2_sf'][e], 32).T
        sample['out'] = acc2.to(torch.bfloat16)
        rows += x_q.shape[0]
    return rows


def time_cpu_sample(sample, steps, warmup):
    import torch
    torch.set_num_threads(os.cpu_count() or 1)
    rows = 0
    for _ in range(warmup):
        rows = cpu_sample_pass(sample)
    t0 = time.perf_counter()
    for _ in range(steps):
        rows = cpu_sample_pass(sample)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return rows, dt, torch.get_num_threads()


def make_cpu_sample_on_cpu(cfg):
    """Seeded CPU-only inputs for the reference arm: rank 0's tokens and router logits of the GPU arm (same generator,
    same order of draws, so the same routed rows), rows of the first CPU_SAMPLE_EXPERTS experts kept; their weights drawn
    ~N(0, 0.02) and quantised to MXFP4 by the oracle (weight values do not change the time)."""
    import torch
    from oracle import moe as omoe
    from oracle import quant
    torch.manual_seed(INPUT_SEED)
    x = torch.randn(cfg['tokens'], cfg['hidden']).bfloat16()
    idx, w = omoe.route_sigmoid_topk(torch.randn(cfg['tokens'], cfg['experts']), cfg['topk'])
    x_q, x_sf = quant.quantize_fp8_per_token(x, 32)
    sample = {k: [] for k in ('x_q', 'x_sf', 'w', 'l1_q', 'l1_sf', 'l2_q', 'l2_sf')}
    for e in range(min(CPU_SAMPLE_EXPERTS, cfg['experts'])):
        tok, slot = torch.nonzero(idx == e, as_tuple=True)
        sample['x_q'].append(x_q[tok])
        sample['x_sf'].append(x_sf[tok])
        sample['w'].append(w[tok, slot])
        q, sf = quant.quantize_fp4_per_token((torch.randn(2 * cfg['inter'], cfg['hidden']) * 0.02).bfloat16(), 32)
        sample['l1_q'].append(q)
        sample['l1_sf'].append(sf)
        q, sf = quant.quantize_fp4_per_token((torch.randn(cfg['hidden'], cfg['inter']) * 0.02).bfloat16(), 32)
        sample['l2_q'].append(q)
        sample['l2_sf'].append(sf)
    return sample


def sample_description(cfg, rows):
    return (f'routed rows of experts 0..{min(CPU_SAMPLE_EXPERTS, cfg["experts"]) - 1} of the same workload ({rows} of '
            f'{cfg["tokens"] * cfg["topk"]} rows), weights dequantised on the fly, torch fp32 matmul; the rate is '
            'extrapolated from this sample to the whole batch')


def cpu_baseline_entry(cfg, rows, dt, cores):
    """tokens/s of the CPU leg: the sampled rows are rows / topk tokens' worth of work."""
    value = rows / cfg['topk'] / dt
    return {'value': value, 'unit': 'tokens/s', 'cores': cores, 'kind': 'port', 'sample': sample_description(cfg, rows),
            'extrapolated': True, 'sample_fraction': rows / float(cfg['tokens'] * cfg['topk'])}


def run_reference(args, cfg, rank, world):
    """CPU restatement of the reference arithmetic (oracle/), all host threads, on a bounded sample."""
    if rank != 0:
        return
    sample = make_cpu_sample_on_cpu(cfg)
    rows, dt, cores = time_cpu_sample(sample, args.steps, args.warmup)
    entry = cpu_baseline_entry(cfg, rows, dt, cores)
    value = entry['value']
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': value, 'unit': 'tokens/s', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dt * 1e3, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': cfg.get('mma', 'fp8xfp4') + ' (fp32 accumulate)', 'data': 'synthetic',
        'config': workload_config(cfg, args.gpus),
        'cpu_baseline': entry,
        'e2e': {'value': value, 'unit': 'tokens/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(cfg, gpus):
    if cfg.get('mma') == 'nvfp4xnvfp4':
        return {'workload': 'NVFP4 prefill variant of the MoE layer (BASELINE config 4)' + ('' if gpus == 1 else f', {gpus}-GPU expert-parallel'),
                'tokens_per_rank': cfg['tokens'], 'hidden': cfg['hidden'], 'intermediate': cfg['inter'],
                'experts': cfg['experts'], 'topk': cfg['topk'],
                'activations': 'nvfp4 e2m1, 1x16 ue4m3 + fp32 tensor scale (calibrated, fixed)',
                'weights': 'nvfp4 e2m1, 1x16 ue4m3 + fp32 scale per expert matrix',
                'l2_policy': 'inputs larger than L2 (about 8 GB of expert weights streamed every step)'}
    name = ('single-GPU full MoE layer, MXFP4 weights (BASELINE config 3)' if gpus == 1 else
            f'{gpus}-GPU expert-parallel MoE layer, MXFP4 weights (BASELINE config 5)')
    return {'workload': name, 'tokens_per_rank': cfg['tokens'], 'hidden': cfg['hidden'],
            'intermediate': cfg['inter'], 'experts': cfg['experts'], 'topk': cfg['topk'],
            'activations': 'fp8 e4m3, 1x32 ue8m0', 'weights': 'mxfp4 e2m1, 1x32 ue8m0',
            'l2_policy': 'inputs larger than L2 (about 6 GB of expert weights streamed every step)'}


def build_layer(dg, cfg, keep_cpu_experts):
    """Random expert weights ~N(0, 0.02), quantised to MXFP4 on the GPU expert by expert (bounds memory), packed and
    transformed for the layer. Returns (l1, l2, cpu copies of the first `keep_cpu_experts` experts' quantised weights)."""
    import torch
    e, h, i = cfg['local_experts'], cfg['hidden'], cfg['inter']
    l1_q = torch.empty((e, 2 * i, h // 2), dtype=torch.int8, device='cuda')
    l1_sf = torch.empty((e, 2 * i, h // 32), dtype=torch.float32, device='cuda')
    l2_q = torch.empty((e, h, i // 2), dtype=torch.int8, device='cuda')
    l2_sf = torch.empty((e, h, i // 32), dtype=torch.float32, device='cuda')
    for g in range(e):
        w = torch.randn(2 * i, h, device='cuda', dtype=torch.bfloat16) * 0.02
        l1_q[g], l1_sf[g] = dg.utils.per_token_cast_to_fp4(w, use_ue8m0=True, gran_k=32)
        w = torch.randn(h, i, device='cuda', dtype=torch.bfloat16) * 0.02
        l2_q[g], l2_sf[g] = dg.utils.per_token_cast_to_fp4(w, use_ue8m0=True, gran_k=32)
    cpu = {k: [t[g].cpu() for g in range(keep_cpu_experts)]
           for k, t in (('l1_q', l1_q), ('l1_sf', l1_sf), ('l2_q', l2_q), ('l2_sf', l2_sf))}
    l1_sf_p = dg.transform_sf_into_required_layout(l1_sf, 2 * i, h, (1, 32), e)
    l2_sf_p = dg.transform_sf_into_required_layout(l2_sf, h, i, (1, 32), e)
    del l1_sf, l2_sf
    l1, l2 = dg.transform_weights_for_mega_moe((l1_q, l1_sf_p), (l2_q, l2_sf_p))
    del l1_q, l1_sf_p
    torch.cuda.empty_cache()
    return l1, l2, cpu


def build_layer_nvfp4(dg, cfg):
    """Random expert weights ~N(0, 0.02) quantised to NVFP4 on the GPU expert by expert, scales packed MN-major."""
    import torch
    e, h, i = cfg['local_experts'], cfg['hidden'], cfg['inter']
    l1_q = torch.empty((e, 2 * i, h // 2), dtype=torch.int8, device='cuda')
    l1_sf = torch.empty((e, h // 64, 2 * i), dtype=torch.int32, device='cuda').transpose(1, 2)
    l2_q = torch.empty((e, h, i // 2), dtype=torch.int8, device='cuda')
    l2_sf = torch.empty((e, i // 64, h), dtype=torch.int32, device='cuda').transpose(1, 2)
    l1_s = torch.empty(e, dtype=torch.float32, device='cuda')
    l2_s = torch.empty(e, dtype=torch.float32, device='cuda')
    for g in range(e):
        w = torch.randn(2 * i, h, device='cuda', dtype=torch.bfloat16) * 0.02
        l1_q[g], sf, l1_s[g] = dg.per_token_cast_to_nvfp4(w, sf_layout='mn')
        l1_sf[g].copy_(sf)
        w = torch.randn(h, i, device='cuda', dtype=torch.bfloat16) * 0.02
        l2_q[g], sf, l2_s[g] = dg.per_token_cast_to_nvfp4(w, sf_layout='mn')
        l2_sf[g].copy_(sf)
    l1, l2 = dg.transform_weights_for_mega_moe((l1_q, l1_sf, l1_s), (l2_q, l2_sf, l2_s))
    del l1_q, l1_sf
    torch.cuda.empty_cache()
    return l1, l2


def run_gemm_workload(args):
    print(json.dumps(measure_gemm_workload(args.workload == 'gemm_masked', args.steps, args.warmup)), flush=True)


def measure_gemm_workload(masked, steps, warmup):
    """BASELINE configs 1 (m-grouped contiguous, 4 experts, N 512, K 1024) and 2 (masked decode GEMM, 32 experts,
    Poisson(64) rows, N 4096, K 7168), FP8 1x128 activations x MXFP4 1x32 weights, bf16 output. Every timed launch is
    preceded by a 512 MB write that flushes L2; times are per-launch CUDA events."""
    import torch
    import deepgemm_b200 as dg
    from deepgemm_b200 import _lib
    torch.manual_seed(0)
    g, n, k = (32, 4096, 7168) if masked else (4, 512, 1024)
    w_q = torch.empty((g, n, k // 2), dtype=torch.int8, device='cuda')
    w_sf = torch.empty((g, n, k // 32), dtype=torch.float32, device='cuda')
    for e in range(g):
        w_q[e], w_sf[e] = dg.utils.per_token_cast_to_fp4(torch.randn(n, k, device='cuda', dtype=torch.bfloat16) * 0.02,
                                                         use_ue8m0=True, gran_k=32)
    w_sf = dg.transform_sf_into_required_layout(w_sf, n, k, (1, 32), g)  # packed once, as a deployment would
    if masked:
        max_m = 256
        counts = torch.poisson(torch.full((g,), 64.0)).clamp(0, max_m).to(torch.int32)
        a = torch.randn(g * max_m, k, device='cuda', dtype=torch.bfloat16)
        a_q, a_sf = dg.utils.per_token_cast_to_fp8(a, use_ue8m0=True, gran_k=128)
        a_q = a_q.view(g, max_m, k)
        a_sf = dg.transform_sf_into_required_layout(a_sf.view(g, max_m, k // 128), max_m, k, (1, 128), g)
        d = torch.empty((g, max_m, n), dtype=torch.bfloat16, device='cuda')
        layout = counts.cuda()
        rows = int(counts.sum())
        call = lambda: dg.m_grouped_fp8_fp4_gemm_nt_masked((a_q, a_sf), (w_q, w_sf), d, layout, 64, recipe_a=(1, 128), recipe_b=(1, 32))
    else:
        ms = torch.randint(64, 257, (g,))
        aligned = (ms + 127) // 128 * 128
        m = int(aligned.sum())
        row_ids = torch.full((m,), -1, dtype=torch.int32)
        start = 0
        for e in range(g):
            row_ids[start:start + int(ms[e])] = e
            start += int(aligned[e])
        a = torch.randn(m, k, device='cuda', dtype=torch.bfloat16)
        a_q, a_sf = dg.utils.per_token_cast_to_fp8_mn_major(a, gran_k=128)
        d = torch.empty((m, n), dtype=torch.bfloat16, device='cuda')
        layout = row_ids.cuda()
        rows = int(ms.sum())
        call = lambda: dg.m_grouped_fp8_fp4_gemm_nt_contiguous((a_q, a_sf), (w_q, w_sf), d, layout, recipe_a=(1, 128), recipe_b=(1, 32))
    flush = torch.empty(512 << 20, dtype=torch.int8, device='cuda')
    for _ in range(max(warmup, 3)):
        call()
    torch.cuda.synchronize()
    sampler = make_clock_sampler(torch.cuda.current_device())
    sampler.start()
    sampler.begin()
    total = 0.0
    for _ in range(steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        call()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    clocks = sampler.stop()
    _lib.device_status()
    ms_per = total / steps
    peak, peak_kind = measured_peaks()
    flops = 2.0 * rows * n * k
    touched = g if not masked else int((counts > 0).sum())
    nbytes = touched * (n * k // 2 + n * k // 32) + rows * (k + k // 128 + 2 * n)
    return {
        'metric': 'grouped_gemm_us', 'value': ms_per * 1e3, 'unit': 'us', 'n_gpus': 1, 'steps': steps, 'warmup': warmup,
        'ms_per_step': ms_per, 'higher_is_better': False, 'scaling': 'weak', 'vs_baseline': None,
        'dtype': 'fp8xfp4 (fp32 accumulate)', 'data': 'synthetic',
        'config': {'workload': ('m-grouped masked FP8xMXFP4 decode GEMM (BASELINE config 2)' if masked else
                                'm-grouped contiguous FP8xMXFP4 GEMM (BASELINE config 1)'),
                   'groups': g, 'n': n, 'k': k, 'valid_rows': rows, 'l2_policy': 'L2 flushed by a 512 MB write before every launch'},
        'gpu_launches': steps, 'clocks': clocks, 'tflops': flops / (ms_per * 1e-3) / 1e12,
        'roofline': {'kernel': 'dgb200_grouped_gemm_kernel', 'bound': 'hbm', 'achieved': nbytes / (ms_per * 1e-3) / 1e9, 'peak': peak,
                     'unit': 'GB/s', 'frac': nbytes / (ms_per * 1e-3) / 1e9 / peak, 'peak_source': peak_kind, 'traffic': None,
                     'algorithmic_bytes': nbytes},
    }


def measured_bf16_tflops():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)['bf16_tflops']), 'measured'
    return 1590.0, 'fallback'


def run_family_workload(args):
    """Stand-alone timings of the operators next to the headline path: the BF16 family and the K-grouped FP8 GEMM.
    Shapes: bf16_gemm_contiguous 8 groups x 4096 rows, N 4096, K 7168; bf16_gemm_masked 32 groups x 64 of 256 rows, N 4096,
    K 7168; bf16_gemm_dense 8192^3; bf16_layer 4096 tokens, 64 experts, top-8, hidden 7168, intermediate 2048;
    k_grouped_gemm 8 groups, m 4096, n 7168, 4096 K rows per group (FP32 accumulation into d). Inputs are larger than L2
    except where a 512 MB flush is stated; times are CUDA events over all timed launches."""
    import torch
    import deepgemm_b200 as dg
    from deepgemm_b200 import _lib
    torch.manual_seed(0)
    w = args.workload
    hbm_peak, hbm_kind = measured_peaks()
    tf_peak, tf_kind = measured_bf16_tflops()
    bound, flops, nbytes, dtype, extra = 'tensor', 0.0, 0.0, 'bf16 (fp32 accumulate)', {}
    rb = lambda *shape: torch.randn(*shape, device='cuda').bfloat16()
    if w == 'bf16_gemm_contiguous':
        g, mg, n, k = 8, 4096, 4096, 7168
        a, b, d = rb(g * mg, k), rb(g, n, k), torch.empty(g * mg, n, device='cuda', dtype=torch.bfloat16)
        layout = torch.arange(g, device='cuda', dtype=torch.int32).repeat_interleave(mg)
        call = lambda: dg.m_grouped_bf16_gemm_nt_contiguous(a, b, d, layout)
        flops, nbytes = 2.0 * g * mg * n * k, 2.0 * (a.numel() + b.numel() + d.numel())
        extra = {'groups': g, 'rows_per_group': mg, 'n': n, 'k': k}
    elif w == 'bf16_gemm_masked':
        g, mm, n, k, rows = 32, 256, 4096, 7168, 64
        a, b, d = rb(g, mm, k), rb(g, n, k), torch.empty(g, mm, n, device='cuda', dtype=torch.bfloat16)
        masked = torch.full((g,), rows, device='cuda', dtype=torch.int32)
        call = lambda: dg.m_grouped_bf16_gemm_nt_masked(a, b, d, masked, rows)
        bound, flops = 'hbm', 2.0 * g * rows * n * k
        nbytes = 2.0 * (b.numel() + g * rows * (k + n))
        extra = {'groups': g, 'valid_rows_per_group': rows, 'n': n, 'k': k}
    elif w == 'bf16_gemm_dense':
        m = n = k = 8192
        a, b, d = rb(m, k), rb(n, k), torch.empty(m, n, device='cuda', dtype=torch.bfloat16)
        call = lambda: dg.bf16_gemm_nt(a, b, d)
        flops, nbytes = 2.0 * m * n * k, 2.0 * (a.numel() + b.numel() + d.numel())
        extra = {'m': m, 'n': n, 'k': k}
    elif w == 'bf16_layer':
        t, h, i, e, topk = 4096, 7168, 2048, 64, 8
        buf = dg.get_symm_buffer_for_mega_moe(None, e, t, topk, h, i, mma_type='bf16xbf16')
        buf.x.copy_(rb(t, h))
        dg.route_sigmoid_topk(torch.randn(t, e, device='cuda'), topk, buf.topk_idx, buf.topk_weights)
        w1 = (torch.randn(e, 2 * i, h, device='cuda') * 0.02).bfloat16()
        l1, l2 = dg.transform_weights_for_mega_moe(w1, (torch.randn(e, h, i, device='cuda') * 0.02).bfloat16())
        del w1
        y = torch.empty(t, h, device='cuda', dtype=torch.bfloat16)
        call = lambda: dg.bf16_mega_moe(y, l1, l2, buf)
        flops = 2.0 * t * topk * h * i * 3
        nbytes = 2.0 * (l1.numel() + l2.numel()) + t * topk * (2 * h * 2 + 2 * i * 2) + t * h * 2 * (2 + topk)
        extra = {'tokens': t, 'hidden': h, 'intermediate': i, 'experts': e, 'topk': topk, 'tokens_per_s': None}
    else:  # k_grouped_gemm
        g, m, n, kg = 8, 4096, 7168, 4096
        ks = [kg] * g
        a = torch.randn(g * kg, m, device='cuda').to(torch.float8_e4m3fn)
        b = torch.randn(g * kg, n, device='cuda').to(torch.float8_e4m3fn)
        sfa, sfb = torch.ones(g * kg // 128, m, device='cuda'), torch.ones(g * kg // 128, n, device='cuda')
        d = torch.zeros(g, m, n, device='cuda')
        layout = torch.tensor(ks, dtype=torch.int32, device='cuda')
        call = lambda: dg.k_grouped_fp8_gemm_tn_contiguous((a, sfa), (b, sfb), d, ks, layout, c=d)
        flops, nbytes = 2.0 * g * kg * m * n, float(a.numel() + b.numel() + 2 * d.numel() * 4)
        dtype, tf_peak, tf_kind = 'fp8 e4m3 (fp32 accumulate)', 4500.0, 'nominal dense FP8'
        extra = {'groups': g, 'm': m, 'n': n, 'k_per_group': kg}
    for _ in range(max(args.warmup, 3)):
        call()
    torch.cuda.synchronize()
    sampler = make_clock_sampler(0)
    sampler.start()
    sampler.begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        call()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    status = _lib.device_status()
    assert status[0] == 0, status
    ms_per = e0.elapsed_time(e1) / args.steps
    tflops = flops / (ms_per * 1e-3) / 1e12
    gbs = nbytes / (ms_per * 1e-3) / 1e9
    if 'tokens_per_s' in extra:
        extra['tokens_per_s'] = extra['tokens'] / (ms_per * 1e-3)
    extra['workload'] = w
    extra['l2_policy'] = 'inputs larger than L2'
    roofline = ({'bound': 'hbm', 'achieved': gbs, 'peak': hbm_peak, 'unit': 'GB/s', 'frac': gbs / hbm_peak, 'peak_source': hbm_kind}
                if bound == 'hbm' else
                {'bound': 'tensor', 'achieved': tflops, 'peak': tf_peak, 'unit': 'TFLOP/s', 'frac': tflops / tf_peak, 'peak_source': tf_kind})
    roofline.update({'kernel': 'dgb200_grouped_gemm_kernel', 'traffic': None, 'algorithmic_bytes': nbytes})
    print(json.dumps({
        'metric': 'kernel_us', 'value': ms_per * 1e3, 'unit': 'us', 'n_gpus': 1, 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': ms_per, 'higher_is_better': False, 'scaling': 'weak', 'vs_baseline': None, 'dtype': dtype,
        'data': 'synthetic', 'config': extra, 'gpu_launches': args.steps, 'clocks': clocks, 'tflops': tflops, 'gbs': gbs,
        'roofline': roofline,
    }), flush=True)


def ep_parity_check(dg, _lib, rank, world, guests):
    """Correctness of the expert-parallel path at this world size, run after the timed regions: one small layer on every
    rank (256 tokens per rank, hidden 512, intermediate 256, 8 experts per rank, top-4, 15 % masked slots, one shared
    expert, routing biased towards two experts of rank 0 so that, with `guests` guest slots per rank, rows of hot experts
    spill to other ranks), all ranks' outputs and dispatch plans gathered to rank 0 and compared with the CPU oracle
    (checker only).
    The check mirrors the reference's fused-against-baseline comparison (tests/test_mega_moe.py:316-329).
    Returns {'calc_diff_max', 'plan_bit_exact', 'ranks', 'ok'} on rank 0, None elsewhere."""
    import torch
    import torch.distributed as dist
    tokens, hidden, inter, topk, per_rank = 256, 512, 256, 4, 8
    experts = per_rank * world

    def inputs_of(r):
        # the same weights on every rank, tokens and routing seeded by the rank
        from oracle import moe as omoe
        from oracle import quant
        g = torch.Generator().manual_seed(9100 + r)
        x = torch.randn(tokens, hidden, generator=g).bfloat16()
        logits = torch.randn(tokens, experts, generator=g)
        logits[:, :2] += 2.0
        idx, w = omoe.route_sigmoid_topk(logits, topk)
        mask = torch.rand(idx.shape, generator=g) < 0.15
        idx, w = idx.masked_fill(mask, -1), w.masked_fill(mask, 0.0)
        x_q, x_sf = quant.quantize_fp8_per_token(x, 32)
        return dict(x_q=x_q, x_sf=x_sf, topk_idx=idx, topk_weights=w)

    def weights():
        from oracle import quant
        g = torch.Generator().manual_seed(9001)
        out = {}
        for name, shape in (('l1', (experts, 2 * inter, hidden)), ('l2', (experts, hidden, inter))):
            qs, sfs = zip(*[quant.quantize_fp4_per_token((torch.randn(*shape[1:], generator=g) * 0.02).bfloat16(), 32)
                            for _ in range(experts)])
            out[name + '_q'], out[name + '_sf'] = torch.stack(qs), torch.stack(sfs)
        out['s1_q'], out['s1_sf'] = quant.quantize_fp8_per_token((torch.randn(2 * inter, hidden, generator=g) * 0.02).bfloat16(), 32)
        out['s2_q'], out['s2_sf'] = quant.quantize_fp8_per_token((torch.randn(hidden, inter, generator=g) * 0.02).bfloat16(), 32)
        return out

    from oracle import quant
    c, wt = inputs_of(rank), weights()
    mine = slice(rank * per_rank, (rank + 1) * per_rank)
    buf = dg.get_symm_buffer_for_mega_moe(dist.group.WORLD, experts, tokens, topk, hidden, inter, num_shared_experts=1)
    l1_sf = dg.transform_sf_into_required_layout(wt['l1_sf'][mine].cuda(), 2 * inter, hidden, (1, 32), per_rank)
    l2_sf = dg.transform_sf_into_required_layout(wt['l2_sf'][mine].cuda(), hidden, inter, (1, 32), per_rank)
    l1, l2 = dg.transform_weights_for_mega_moe((wt['l1_q'][mine].cuda(), l1_sf), (wt['l2_q'][mine].cuda(), l2_sf))
    if guests > 0:
        l1, l2 = dg.share_weights_for_mega_moe(dist.group.WORLD, l1, l2, num_guest_experts=guests)
    sl1, sl2 = dg.transform_weights_for_mega_moe(
        (wt['s1_q'].cuda(), dg.transform_sf_into_required_layout(wt['s1_sf'].cuda(), 2 * inter, hidden, (1, 32))),
        (wt['s2_q'].cuda(), dg.transform_sf_into_required_layout(wt['s2_sf'].cuda(), hidden, inter, (1, 32))))
    buf.x[:tokens].copy_(c['x_q'].cuda())
    buf.x_sf[:tokens].copy_(quant.pack_ue8m0(c['x_sf']).cuda())
    buf.topk_idx[:tokens].copy_(c['topk_idx'].cuda())
    buf.topk_weights[:tokens].copy_(c['topk_weights'].cuda())
    y = torch.full((tokens, hidden), float('nan'), dtype=torch.bfloat16, device='cuda')
    dg.fp8_fp4_mega_moe(y, l1, l2, buf, shared_l1_weights=sl1, shared_l2_weights=sl2)
    status = _lib.device_status(raise_on_error=False)
    lay = buf.layout
    slots = per_rank + guests
    plan = torch.cat([buf.buffer[lay[k]:lay[k] + n * 4].view(torch.int32) for k, n in
                      (('expert_start', slots), ('expert_end', slots), ('dest_row', tokens * topk), ('my_dest', experts),
                       ('my_slot', experts), ('guest_expert', guests))])
    ys = [torch.empty_like(y) for _ in range(world)]
    plans = [torch.empty_like(plan) for _ in range(world)]
    codes = [torch.zeros(1, dtype=torch.int32, device='cuda') for _ in range(world)]
    dist.all_gather(ys, y)
    dist.all_gather(plans, plan)
    dist.all_gather(codes, torch.tensor([status[0]], dtype=torch.int32, device='cuda'))
    if rank != 0:
        return None
    from oracle import moe as omoe
    cases = [inputs_of(r) for r in range(world)]
    all_counts = torch.stack([omoe.ep_counts(cs['topk_idx'], experts) for cs in cases])
    diff_max, plan_ok, spilled = 0.0, True, 0
    for r in range(world):
        cs = cases[r]
        shared = omoe.shared_expert_rows(cs['x_q'], cs['x_sf'], wt['s1_q'], wt['s1_sf'], wt['s2_q'], wt['s2_sf'])
        want = omoe.moe_layer(cs['x_q'], cs['x_sf'], cs['topk_idx'], cs['topk_weights'], wt['l1_q'], wt['l1_sf'], wt['l2_q'],
                              wt['l2_sf'], shared_rows=shared)
        got = ys[r].cpu()
        d = float(quant.calc_diff(got, want)) if not torch.isnan(got.float()).any() else float('inf')
        diff_max = max(diff_max, d)
        p = plans[r].cpu().long()
        if guests > 0:
            my_base, my_dest, my_slot, want_start, want_end, guest = omoe.ep_plan_with_spill(all_counts, r, 128, guests)
            spilled += int((guest >= 0).sum())
            want_plan = torch.cat([want_start, want_end, omoe.ep_dest_rows(cs['topk_idx'], my_base, experts).long(), my_dest, my_slot, guest])
        else:
            my_base, want_start, want_end = omoe.ep_plan(all_counts, r, 128)
            want_plan = torch.cat([want_start, want_end, omoe.ep_dest_rows(cs['topk_idx'], my_base, experts).long(), p[2 * slots + tokens * topk:]])
        plan_ok = plan_ok and torch.equal(p, want_plan)
    status_ok = all(int(cd) == 0 for cd in codes)
    return {'calc_diff_max': diff_max, 'plan_bit_exact': bool(plan_ok), 'device_status_ok': status_ok, 'ranks': world,
            'tolerance': 2e-3, 'ok': bool(plan_ok and status_ok and diff_max <= 2e-3), 'guest_slots_per_rank': guests,
            'experts_spilled': spilled,
            'case': f'{tokens} tokens/rank, hidden {hidden}, inter {inter}, {experts} experts, top-{topk}, 15% masked, 1 shared expert'}


def layer_line(args, cfg, rank, world, local_rank, steps, warmup, with_e2e=True, with_cpu=True, weights=None):
    """Builds (or reuses) the layer's weights, times `steps` passes after `warmup` untimed ones and returns, on rank 0,
    the JSON line as a dict plus the weights (None and the weights on the other ranks)."""
    import torch
    import torch.distributed as dist
    import deepgemm_b200 as dg
    from deepgemm_b200 import _lib

    torch.cuda.set_device(local_rank)
    torch.manual_seed(INPUT_SEED + rank)
    t, h, i, e, k = cfg['tokens'], cfg['hidden'], cfg['inter'], cfg['experts'], cfg['topk']
    cfg['local_experts'] = e // world
    nvfp4 = cfg.get('mma') == 'nvfp4xnvfp4'
    with_cpu = with_cpu and rank == 0 and world == 1 and not nvfp4 and not args.skip_cpu_baseline
    # the first CPU draws of this function are the tokens and the logits, in this order: the reference arm repeats them
    x_host = torch.randn(t, h).bfloat16().pin_memory()
    logits = torch.randn(t, e)
    cpu_weights = None
    if weights is not None:
        l1, l2 = weights
    elif nvfp4:
        l1, l2 = build_layer_nvfp4(dg, cfg)
    else:
        l1, l2, cpu_weights = build_layer(dg, cfg, min(CPU_SAMPLE_EXPERTS, e) if with_cpu else 0)
    if nvfp4:
        # calibrated, fixed scales (equal on every rank): inputs ~N(0, 1) stay below 8; post-SwiGLU values below 64
        x_scale = torch.tensor(8.0 / (6 * 448), device='cuda')
        act_scale = torch.tensor(64.0 / (6 * 448), device='cuda')
    guests = args.guest_experts if world > 1 and not nvfp4 else 0
    if guests > 0:
        # hot experts may spill rows to other ranks: the weights move into symmetric memory with room for guest experts
        l1, l2 = dg.share_weights_for_mega_moe(dist.group.WORLD, l1, l2, num_guest_experts=guests)
    buf = dg.get_symm_buffer_for_mega_moe(dist.group.WORLD if world > 1 else None, e, t, k, h, i, mma_type=cfg.get('mma', 'fp8xfp4'))
    if world > 1:
        # expert popularity ~ Zipf(s = 1): rank r of a seeded random permutation of the experts has weight 1 / (r + 1)
        g = torch.Generator().manual_seed(2024)
        popularity = torch.empty(e)
        popularity[torch.randperm(e, generator=g)] = 1.0 / torch.arange(1, e + 1, dtype=torch.float32)
        logits = logits + torch.log(popularity / popularity.sum())
    logits_host = logits.pin_memory()
    y_host = torch.empty((t, h), dtype=torch.bfloat16).pin_memory()
    x = x_host.cuda()
    logits = logits_host.cuda()
    y = torch.empty((t, h), dtype=torch.bfloat16, device='cuda')
    lib = _lib.lib()
    kernels_per_step = kernels_of_one_step(nvfp4, world, cfg['local_experts'], guests, args.comm_sms)

    def step(events=None, x_in=None, logits_in=None, y_out=None):
        x_in, logits_in, y_out = (x if x_in is None else x_in), (logits if logits_in is None else logits_in), (y if y_out is None else y_out)
        if events is not None:
            arr = (ctypes.c_void_p * len(events))(*[None if ev is None else ev.cuda_event for ev in events])
            _lib.check(lib.dgb200_set_mega_moe_stage_events(ctypes.cast(arr, ctypes.c_void_p), len(events)))
        if nvfp4 and world == 1:
            # router -> dispatch plan -> BF16 rows quantised to NVFP4 while they are dispatched -> L1 -> L2 -> combine
            dg.nvfp4_mega_moe_bf16_input(y_out, x_in, l1, l2, buf, x_scale, act_scale, logits=logits_in)
        elif nvfp4:
            dg.route_sigmoid_topk(logits_in, k, buf.topk_idx, buf.topk_weights)
            dg.per_token_cast_to_nvfp4_into(x_in, x_scale, buf.x, buf.x_sf)
            dg.nvfp4_mega_moe(y_out, l1, l2, buf, x_scale, act_scale)
        else:
            # router -> dispatch plan -> BF16 rows quantised to FP8 while they are dispatched -> L1 -> L2 -> combine
            dg.fp8_fp4_mega_moe_bf16_input(y_out, x_in, l1, l2, buf, logits=logits_in)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    sampler = make_clock_sampler(local_rank)
    sampler.start()
    barrier()
    for _ in range(warmup):
        step()
    barrier()
    _lib.device_status()
    stage_events = [[torch.cuda.Event(enable_timing=True) for _ in range(6)] for _ in range(steps)]
    for evs in stage_events:  # create the underlying handles before they are handed to the library
        for ev in evs:
            ev.record()
    barrier()
    # The timed steps carry only the two events around the roofline kernel (the gate/up GEMM stage; expert parallel: all
    # GEMMs): an event between two kernels serialises their launches, so the full stage breakdown comes from a second pass
    # of the same steps that is not part of the timed region.
    roof_a, roof_b = 2, 3
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.begin()
    t0.record()
    for s in range(steps):
        step(None if args.no_stage_events else [ev if j in (roof_a, roof_b) else None for j, ev in enumerate(stage_events[s])])
    t1.record()
    barrier()
    sampler.end()
    clocks = sampler.stop()
    ms_per_step = t0.elapsed_time(t1) / steps
    _lib.device_status()
    if args.no_stage_events:
        stage_ms, roof_ms = [float('nan')] * 5, float('nan')
    else:
        roof_ms = sum(evs[roof_a].elapsed_time(evs[roof_b]) for evs in stage_events) / steps
        for s in range(steps):
            step(stage_events[s])
        barrier()
        _lib.device_status()
        stage_ms = [sum(evs[j].elapsed_time(evs[j + 1]) for evs in stage_events) / steps for j in range(5)]

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region.
    # Every step copies its own inputs from pinned host memory and its result back; the three legs run on three
    # streams over double-buffered device staging, so step s + 1's upload and step s - 1's download overlap step s.
    e2e_ms = float('nan')
    if with_e2e:
        compute = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        xs, lgs, ys = [x, torch.empty_like(x)], [logits, torch.empty_like(logits)], [y, torch.empty_like(y)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def e2e_steps(n):
            for s in range(n):
                slot = s & 1
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_done[slot])   # the step that last read this slot's inputs has finished
                    xs[slot].copy_(x_host, non_blocking=True)
                    lgs[slot].copy_(logits_host, non_blocking=True)
                    ev_in[slot].record(s_in)
                compute.wait_event(ev_in[slot])
                compute.wait_event(ev_out[slot])     # this slot's previous result has left the device
                step(None, xs[slot], lgs[slot], ys[slot])
                ev_done[slot].record(compute)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[slot])
                    y_host.copy_(ys[slot], non_blocking=True)
                    ev_out[slot].record(s_out)
            compute.wait_event(ev_out[0])
            compute.wait_event(ev_out[1])

        e2e_steps(max(warmup, 3))
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_steps(steps)
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / steps
        _lib.device_status()

    # ---- algorithmic work of this batch, per rank
    lay = buf.layout
    slots = cfg['local_experts'] + guests  # guest slots follow the rank's own experts
    ends = buf.buffer[lay['expert_end']:lay['expert_end'] + slots * 4].view(torch.int32).cpu()
    starts = buf.buffer[lay['expert_start']:lay['expert_start'] + slots * 4].view(torch.int32).cpu()
    rows = int((ends - starts).sum())
    touched = int(((ends - starts) > 0).sum())
    rows_before_spill = spilled_experts = None
    if guests > 0:
        rows_before_spill = buf.buffer[lay['rank_rows']:lay['rank_rows'] + world * 4].view(torch.int32).cpu().tolist()
        hosted = buf.buffer[lay['guest_expert']:lay['guest_expert'] + guests * 4].view(torch.int32).cpu()
        spilled_experts = int((hosted >= 0).sum())
    if nvfp4:
        l1_bytes = touched * (2 * i * h // 2 + 2 * i * h // 16) + rows * (h // 2 + h // 16) + rows * (i // 2 + i // 16)
        l2_bytes = touched * (h * i // 2 + h * i // 16) + rows * (i // 2 + i // 16) + rows * h * 2
    else:
        l1_bytes = touched * (2 * i * h // 2 + 2 * i * h // 32) + rows * (h + h // 32) + rows * (i + i // 32)
        l2_bytes = touched * (h * i // 2 + h * i // 32) + rows * (i + i // 32) + rows * h * 2
    # every rank's own numbers travel to rank 0: the step time is the maximum over ranks, everything that explains it
    # (stage times, bytes, flops) is taken from ONE rank, the one with the most routed rows
    mine = torch.tensor([ms_per_step, e2e_ms] + stage_ms + [rows, touched, l1_bytes, l2_bytes, spilled_experts or 0, roof_ms],
                        dtype=torch.float64, device='cuda')
    per_rank = [torch.empty_like(mine) for _ in range(world)]
    if world > 1:
        dist.all_gather(per_rank, mine)
    else:
        per_rank = [mine]
    if rank != 0:
        return None, (l1, l2)
    table = torch.stack(per_rank).cpu()
    ms_per_step, e2e_ms = float(table[:, 0].max()), float(table[:, 1].max())
    hot = int(table[:, 7].argmax())
    stage_ms = [float(v) for v in table[hot, 2:7]]
    roof_ms = float(table[hot, 12])  # the roofline kernel's interval inside the timed steps, same rank
    rows_hot, l1_bytes, l2_bytes = int(table[hot, 7]), int(table[hot, 9]), int(table[hot, 10])
    rows_all = float(table[:, 7].sum())
    flops = 2.0 * rows_all * h * i * 3
    hbm_peak, peak_kind = measured_peaks()
    tflops = flops / (ms_per_step * 1e-3) / 1e12
    # dominant kernel = the gate/up GEMM of the most loaded rank; which roofline binds it follows from its arithmetic
    # intensity against the ridge of the FP8 tensor rate (nominal; this pool has no measured FP8 figure) over HBM
    l1_flops = 2.0 * rows_hot * h * 2 * i
    l1_s = roof_ms * 1e-3
    gemms_in_one_interval = world > 1  # expert parallel: gate/up and down GEMMs alternate phase by phase
    if gemms_in_one_interval:
        l1_flops = 2.0 * rows_hot * h * 3 * i
        l1_bytes = l1_bytes + l2_bytes
    mma_peak_nominal = FP4_DENSE_PEAK_TFLOPS_NOMINAL if nvfp4 else FP8_DENSE_PEAK_TFLOPS_NOMINAL
    tensor_bound = l1_bytes > 0 and l1_flops / l1_bytes > mma_peak_nominal * 1e12 / (hbm_peak * 1e9)
    l1_kernel_name = ('dgb200_grouped_gemm_kernel (gate/up + SwiGLU + requant and down GEMMs of all expert phases, with the waits for '
                      'the other ranks\' rows between them)' if world > 1 else
                      'dgb200_grouped_gemm_kernel (gate/up GEMM + SwiGLU + requant)' if nvfp4 else L1_STAGE_KERNELS)
    if tensor_bound:
        roofline = {'kernel': l1_kernel_name, 'bound': 'tensor', 'achieved': l1_flops / l1_s / 1e12, 'peak': mma_peak_nominal,
                    'unit': 'TFLOP/s', 'frac': l1_flops / l1_s / 1e12 / mma_peak_nominal,
                    'peak_source': 'nominal dense ' + ('FP4' if nvfp4 else 'FP8') + ' rate (no measured figure for this type on this pool)',
                    'traffic': None, 'algorithmic_flops': l1_flops, 'algorithmic_bytes': l1_bytes, 'kernel_ms': roof_ms}
    else:
        l1_gbs = l1_bytes / l1_s / 1e9
        roofline = {'kernel': l1_kernel_name, 'bound': 'hbm', 'achieved': l1_gbs, 'peak': hbm_peak, 'unit': 'GB/s',
                    'frac': l1_gbs / hbm_peak, 'peak_source': peak_kind,
                    'traffic': int(L1_KERNEL_DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE * l1_bytes) if not nvfp4 else None,
                    'traffic_source': L1_TRAFFIC_SOURCE if not nvfp4 else None,
                    'algorithmic_bytes': l1_bytes, 'kernel_ms': roof_ms}
    if world > 1:
        roofline['rank'] = hot
    line = {
        'metric': METRIC, 'value': t * world / (ms_per_step * 1e-3), 'unit': 'tokens/s', 'n_gpus': world,
        'steps': steps, 'warmup': warmup, 'ms_per_step': ms_per_step, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': cfg.get('mma', 'fp8xfp4') + ' (fp32 accumulate)', 'data': 'synthetic',
        'config': workload_config(cfg, world),
        'gpu_launches': kernels_per_step * steps,
        'clocks': clocks,
        'roofline': roofline,
        # stage times of the most loaded rank (rank `stages_rank`); with several ranks the cross-rank waits are inside
        'stages_ms': ({'plan': stage_ms[0], 'dispatch': stage_ms[1], 'l1_gemm_swiglu': stage_ms[2],
                       'l2_gemm': stage_ms[3], 'combine': stage_ms[4]} if not gemms_in_one_interval else
                      {'plan': stage_ms[0], 'dispatch_push': stage_ms[1],
                       'gemms_and_return_push': stage_ms[2] + stage_ms[3], 'waits_and_combine': stage_ms[4]}),
        'stages_rank': hot,
        'stages_source': ('a second pass of the same steps with CUDA events at every stage boundary; the timed steps carry only the '
                          'two events around the roofline kernel (roofline.kernel_ms), because an event between two kernels '
                          'serialises their launches'),
        'l2_gemm_hbm_gbs': l2_bytes / (stage_ms[3] * 1e-3) / 1e9 if not gemms_in_one_interval else None,
        'tflops': tflops,
        'frac_fp4_dense_peak_nominal': tflops / (FP4_DENSE_PEAK_TFLOPS_NOMINAL * world),
        'frac_fp8_rate_peak_nominal': tflops / (FP8_DENSE_PEAK_TFLOPS_NOMINAL * world),
        'routed_rows': rows_hot,
        'load_imbalance_max_over_mean': rows_hot / (rows_all / world) if rows_all > 0 else None,
    }
    if world > 1:
        # hot-expert row spill: rows per rank as routed (every expert on its owner) and as computed (above)
        line['hot_expert_spill'] = {
            'guest_slots_per_rank': guests,
            'guest_slots_used': int(table[:, 11].sum()),
            'routing': 'router logits biased by the log of a Zipf(1.0) popularity over a seeded permutation of the experts',
            'return_transfer': ('inside the down GEMM (rows stored to their source ranks from its epilogue)' if guests and args.comm_sms <= 0
                                and args.fused_return != 0 else 'a kernel of its own' if guests else 'pulled by the combine, phase by phase'),
            'load_imbalance_as_routed': (max(rows_before_spill) / (sum(rows_before_spill) / world)) if rows_before_spill else
            line['load_imbalance_max_over_mean'],
        }
    if with_e2e:
        line['e2e'] = {'value': t * world / (e2e_ms * 1e-3), 'unit': 'tokens/s', 'ms_per_step': e2e_ms,
                       'h2d_bytes_per_step': x_host.numel() * 2 + logits_host.numel() * 4, 'd2h_bytes_per_step': y_host.numel() * 2}
    if with_cpu and cpu_weights is not None:
        idx, w = buf.topk_idx[:t].cpu(), buf.topk_weights[:t].cpu()
        from oracle import quant
        x_q_g, x_sf_g = dg.utils.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=32, use_packed_ue8m0=True)
        x_q_c, x_sf_c = x_q_g.cpu(), quant.unpack_ue8m0(x_sf_g.cpu())
        sample = dict(cpu_weights)
        sample.update({'x_q': [], 'x_sf': [], 'w': []})
        for g in range(len(cpu_weights['l1_q'])):
            tok, slot = torch.nonzero(idx == g, as_tuple=True)
            sample['x_q'].append(x_q_c[tok])
            sample['x_sf'].append(x_sf_c[tok])
            sample['w'].append(w[tok, slot])
        srows, dt, cores = time_cpu_sample(sample, 3, 1)
        line['cpu_baseline'] = cpu_baseline_entry(cfg, srows, dt, cores)
    buf.destroy()
    return line, (l1, l2)


def kernels_of_one_step(nvfp4, world, local_experts, guests=0, comm_sms=0):
    """Launches of this library's kernels in one pass of the layer (memsets are not kernels of ours). FP8 layer on one
    rank: router, count, scan, assign, quantise + dispatch, the two GEMMs each split over the two tile orientations
    (2 + 2 launches) plus the SwiGLU finisher, combine; NVFP4: router, count, scan, assign, quantise + dispatch, two GEMMs, combine. Expert parallel, P =
    phases (one with guest experts on one stream, else min(4, expert slots)): router, count, publish counts, flag, plan, assign, quantise, then per phase push + flag,
    flag + scale reorder + L1 + L2, return push + flag, and at the end a flag wait per phase and the combine; with guest
    experts one more launch fetches their weights and the guest slots count as experts."""
    if world == 1:
        return 8 if nvfp4 else 11
    phases = 1 if (guests and comm_sms <= 0) else min(4, local_experts + guests)
    return 7 + 9 * phases + 1 + (1 if guests else 0)


L1_STAGE_KERNELS = ('gate/up GEMM + SwiGLU + FP8 requant (dgb200_grouped_gemm_kernel + dgb200_swap_gemm_kernel + '
                    'dgb200_swiglu_requant_rows_kernel)')


def run_ours(args, cfg, rank, world, local_rank):
    import torch
    import deepgemm_b200 as dg
    from deepgemm_b200 import _lib
    line, weights = layer_line(args, cfg, rank, world, local_rank, args.steps, args.warmup)
    headline = world == 1 and cfg.get('mma') != 'nvfp4xnvfp4' and not args.tokens and not args.experts
    failed = False
    if world > 1:
        parity = ep_parity_check(dg, _lib, rank, world, args.guest_experts if cfg.get('mma') != 'nvfp4xnvfp4' else 0)
        if rank == 0:
            line['ep_parity'] = parity
            failed = not parity['ok']
    elif headline and not args.skip_other_configs:
        # the same layer at 8192 tokens (the per-rank batch of the expert-parallel runs): the like-for-like base of the
        # weak-scaling curve; the headline value above stays BASELINE config 3
        cfg8 = dict(cfg, tokens=8192)
        base, _ = layer_line(args, cfg8, rank, world, local_rank, max(args.steps // 2, 3), 3, with_e2e=False, with_cpu=False, weights=weights)
        line['base_8192_tokens_per_rank'] = {k: base[k] for k in ('value', 'unit', 'ms_per_step', 'stages_ms', 'clocks')}
        del weights
        torch.cuda.empty_cache()
        other = {}
        for name, masked in (('config1_m_grouped_contiguous', False), ('config2_m_grouped_masked', True)):
            other[name] = measure_gemm_workload(masked, max(args.steps, 10), 3)
        cfg4 = dict(cfg, mma='nvfp4xnvfp4', tokens=16384)
        c4, w4 = layer_line(args, cfg4, rank, world, local_rank, max(args.steps // 2, 3), 3, with_e2e=False, with_cpu=False)
        del w4
        other['config4_nvfp4_prefill_layer'] = {k: c4[k] for k in ('value', 'unit', 'ms_per_step', 'tflops', 'frac_fp4_dense_peak_nominal',
                                                                  'stages_ms', 'clocks', 'roofline', 'config')}
        line['other_configs'] = other
    if rank == 0:
        print(json.dumps(line), flush=True)
    return 1 if failed else 0


def keep_stdout_for_the_json_line():
    """Native libraries (NCCL's version banner, for one) write to file descriptor 1 behind Python's back. Point that
    descriptor at stderr and keep the original for sys.stdout, so the one JSON line is all that reaches stdout."""
    sys.stdout.flush()
    kept = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(kept, 'w')


def main():
    args = parse_args()
    keep_stdout_for_the_json_line()
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    cfg = dict(CONFIG3)
    cfg['mma'] = args.mma
    if args.mma == 'nvfp4xnvfp4':
        cfg['tokens'] = 16384
    if args.gpus > 1:
        cfg['tokens'] = 8192
    if args.tokens:
        cfg['tokens'] = args.tokens
    if args.experts:
        cfg['experts'] = args.experts
    if args.workload != 'layer':
        if args.impl == 'reference' or args.gpus != 1:
            raise SystemExit('--workload gemm_* is a single-GPU timing of our kernels only')
        if args.workload in ('gemm_contiguous', 'gemm_masked'):
            run_gemm_workload(args)
        else:
            run_family_workload(args)
        return
    if args.impl == 'reference':
        if args.mma != 'fp8xfp4':
            raise SystemExit('--impl reference times the headline FP8 x MXFP4 workload only')
        run_reference(args, cfg, rank, world)
        return
    if world != args.gpus:
        raise SystemExit(f'--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)')
    if world > 1:
        import torch
        import torch.distributed as dist
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        torch.cuda.set_device(local_rank)
        dist.init_process_group('nccl', device_id=torch.device('cuda', local_rank))
    if args.comm_sms >= 0:
        from deepgemm_b200 import _lib
        _lib.check(_lib.lib().dgb200_set_tuning(b'ep_comm_sms', args.comm_sms))
    if args.pdl >= 0:
        from deepgemm_b200 import _lib
        _lib.check(_lib.lib().dgb200_set_tuning(b'pdl', args.pdl))
    if args.fused_return >= 0:
        from deepgemm_b200 import _lib
        _lib.check(_lib.lib().dgb200_set_tuning(b'fused_return', args.fused_return))
    if args.fused_dispatch >= 0:
        from deepgemm_b200 import _lib
        _lib.check(_lib.lib().dgb200_set_tuning(b'fused_dispatch', args.fused_dispatch))
    rc = run_ours(args, cfg, rank, world, local_rank)
    if world > 1:
        import torch.distributed as dist
        code = torch.tensor([rc], device='cuda')
        dist.broadcast(code, 0)  # every rank leaves with rank 0's outcome of the parity check
        rc = int(code)
        dist.barrier()
        dist.destroy_process_group()
    if rc:
        raise SystemExit(rc)


if __name__ == '__main__':
    main()
