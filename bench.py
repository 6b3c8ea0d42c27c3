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
CPU_SAMPLE_EXPERTS = 4  # experts whose routed rows the CPU legs evaluate per pass
FP4_DENSE_PEAK_TFLOPS_NOMINAL = 9000.0
FP8_DENSE_PEAK_TFLOPS_NOMINAL = 4500.0
# DRAM bytes (read + write) per algorithmic byte of the dominant kernel, from the ncu capture summarised in
# profiles/grouped_gemm_small_layer_ncu_full.md (small case, scaled by the units processed).
L1_KERNEL_DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.06


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--tokens', type=int, default=0, help='override tokens per rank (profiling small cases only)')
    ap.add_argument('--experts', type=int, default=0, help='override the expert count (profiling small cases only)')
    ap.add_argument('--skip-cpu-baseline', action='store_true')
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


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,'
              'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
              'clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.file = tempfile.NamedTemporaryFile('w+', suffix='.csv', delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--query-gpu={self.FIELDS}', '--format=csv,noheader,nounits',
                                          '-lms', '20', '-i', str(self.gpu_index)], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        self.file.flush()
        self.file.seek(0)
        clocks, max_clock, reasons = [], None, set()
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clock = float(parts[2])
            except ValueError:
                continue
            for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), parts[5:9]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        clocks.sort()
        return {'sm_mhz': clocks[len(clocks) // 2] if clocks else None, 'sm_max_mhz': max_clock,
                'samples': len(clocks), 'reasons': sorted(reasons)}


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


def make_cpu_sample_on_cpu(cfg, seed=0):
    """Seeded CPU-only inputs for the reference arm: all tokens routed over all experts, rows of the first
    CPU_SAMPLE_EXPERTS experts kept; their weights drawn ~N(0, 0.02) and quantised to MXFP4 by the oracle."""
    import torch
    from oracle import moe as omoe
    from oracle import quant
    torch.manual_seed(seed)
    x = torch.randn(cfg['tokens'], cfg['hidden']).bfloat16()
    idx, w = omoe.route_sigmoid_topk(torch.randn(cfg['tokens'], cfg['experts']), cfg['topk'])
    x_q, x_sf = quant.quantize_fp8_per_token(x, 32)
    sample = {k: [] for k in ('x_q', 'x_sf', 'w', 'l1_q', 'l1_sf', 'l2_q', 'l2_sf')}
    for e in range(CPU_SAMPLE_EXPERTS):
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
    return (f'routed rows of experts 0..{CPU_SAMPLE_EXPERTS - 1} of the same workload ({rows} of '
            f'{cfg["tokens"] * cfg["topk"]} rows), weights dequantised on the fly, torch fp32 matmul')


def run_reference(args, cfg, rank, world):
    """CPU restatement of the reference arithmetic (oracle/), all host threads, on a bounded sample."""
    if rank != 0:
        return
    sample = make_cpu_sample_on_cpu(cfg)
    rows, dt, cores = time_cpu_sample(sample, args.steps, args.warmup)
    value = rows / cfg['topk'] / dt
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': value, 'unit': 'tokens/s', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dt * 1e3, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': cfg.get('mma', 'fp8xfp4') + ' (fp32 accumulate)', 'data': 'synthetic',
        'config': workload_config(cfg, args.gpus),
        'cpu_baseline': {'value': value, 'unit': 'tokens/s', 'cores': cores, 'kind': 'port',
                         'sample': sample_description(cfg, rows)},
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
    """BASELINE configs 1 (m-grouped contiguous, 4 experts, N 512, K 1024) and 2 (masked decode GEMM, 32 experts,
    Poisson(64) rows, N 4096, K 7168), FP8 1x128 activations x MXFP4 1x32 weights, bf16 output. Every timed launch is
    preceded by a 512 MB write that flushes L2; times are per-launch CUDA events."""
    import torch
    import deepgemm_b200 as dg
    from deepgemm_b200 import _lib
    torch.manual_seed(0)
    masked = args.workload == 'gemm_masked'
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
    for _ in range(max(args.warmup, 3)):
        call()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    total = 0.0
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        call()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    clocks = sampler.stop()
    _lib.device_status()
    ms_per = total / args.steps
    peak, peak_kind = measured_peaks()
    flops = 2.0 * rows * n * k
    touched = g if not masked else int((counts > 0).sum())
    nbytes = touched * (n * k // 2 + n * k // 32) + rows * (k + k // 128 + 2 * n)
    print(json.dumps({
        'metric': 'grouped_gemm_us', 'value': ms_per * 1e3, 'unit': 'us', 'n_gpus': 1, 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': ms_per, 'higher_is_better': False, 'scaling': 'weak', 'vs_baseline': None,
        'dtype': 'fp8xfp4 (fp32 accumulate)', 'data': 'synthetic',
        'config': {'workload': ('m-grouped masked FP8xMXFP4 decode GEMM (BASELINE config 2)' if masked else
                                'm-grouped contiguous FP8xMXFP4 GEMM (BASELINE config 1)'),
                   'groups': g, 'n': n, 'k': k, 'valid_rows': rows, 'l2_policy': 'L2 flushed by a 512 MB write before every launch'},
        'gpu_launches': args.steps, 'clocks': clocks, 'tflops': flops / (ms_per * 1e-3) / 1e12,
        'roofline': {'kernel': 'dgb200_grouped_gemm_kernel', 'bound': 'hbm', 'achieved': nbytes / (ms_per * 1e-3) / 1e9, 'peak': peak,
                     'unit': 'GB/s', 'frac': nbytes / (ms_per * 1e-3) / 1e9 / peak, 'peak_source': peak_kind, 'traffic': None,
                     'algorithmic_bytes': nbytes},
    }), flush=True)


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
    sampler = ClockSampler(0)
    sampler.start()
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


def run_ours(args, cfg, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import deepgemm_b200 as dg
    from deepgemm_b200 import _lib

    torch.cuda.set_device(local_rank)
    torch.manual_seed(1234 + rank)
    t, h, i, e, k = cfg['tokens'], cfg['hidden'], cfg['inter'], cfg['experts'], cfg['topk']
    cfg['local_experts'] = e // world
    nvfp4 = cfg.get('mma') == 'nvfp4xnvfp4'
    if nvfp4:
        args.skip_cpu_baseline = True  # the CPU baseline belongs to the headline workload
        l1, l2 = build_layer_nvfp4(dg, cfg)
        # calibrated, fixed scales (equal on every rank): inputs ~N(0, 1) stay below 8; post-SwiGLU values below 64
        x_scale = torch.tensor(8.0 / (6 * 448), device='cuda')
        act_scale = torch.tensor(64.0 / (6 * 448), device='cuda')
    else:
        l1, l2, cpu_weights = build_layer(dg, cfg, CPU_SAMPLE_EXPERTS if rank == 0 and world == 1 and not args.skip_cpu_baseline else 0)
    buf = dg.get_symm_buffer_for_mega_moe(dist.group.WORLD if world > 1 else None, e, t, k, h, i, mma_type=cfg.get('mma', 'fp8xfp4'))
    x_host = torch.randn(t, h).bfloat16().pin_memory()
    logits = torch.randn(t, e)
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
    # single rank: router, count, scan, assign, quantise + dispatch, L1, L2, combine (the memset is not a kernel of ours);
    # NVFP4 keeps a separate cast and gather; expert parallel adds the count exchange, the plan and three barriers
    # single-rank FP8 layer: both GEMMs are split over the two tile orientations (the library decides from the expected
    # rows per expert), so 2 + 2 GEMM launches and the SwiGLU finisher instead of 2 launches
    kernels_per_step = 9 if nvfp4 else (11 if world == 1 else 12)

    def step(events=None, x_in=None, logits_in=None, y_out=None):
        x_in, logits_in, y_out = (x if x_in is None else x_in), (logits if logits_in is None else logits_in), (y if y_out is None else y_out)
        if events is not None:
            arr = (ctypes.c_void_p * len(events))(*[ev.cuda_event for ev in events])
            _lib.check(lib.dgb200_set_mega_moe_stage_events(ctypes.cast(arr, ctypes.c_void_p), len(events)))
        if nvfp4:
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
    barrier()
    for _ in range(args.warmup):
        step()
    barrier()
    status = _lib.device_status()
    stage_events = [[torch.cuda.Event(enable_timing=True) for _ in range(6)] for _ in range(args.steps)]
    for evs in stage_events:  # create the underlying handles before they are handed to the library
        for ev in evs:
            ev.record()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for s in range(args.steps):
        step(stage_events[s])
    t1.record()
    barrier()
    clocks = sampler.stop()
    ms_per_step = t0.elapsed_time(t1) / args.steps
    status = _lib.device_status()
    stage_ms = [sum(evs[j].elapsed_time(evs[j + 1]) for evs in stage_events) / args.steps for j in range(5)]

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region.
    # Every step copies its own inputs from pinned host memory and its result back; the three legs run on three
    # streams over double-buffered device staging, so step s + 1's upload and step s - 1's download overlap step s.
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

    e2e_steps(max(args.warmup, 3))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_steps(args.steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / args.steps
    _lib.device_status()

    # ---- algorithmic work of this batch
    lay = buf.layout
    ends = buf.buffer[lay['expert_end']:lay['expert_end'] + cfg['local_experts'] * 4].view(torch.int32).cpu()
    starts = buf.buffer[lay['expert_start']:lay['expert_start'] + cfg['local_experts'] * 4].view(torch.int32).cpu()
    rows = int((ends - starts).sum())
    rows_all = torch.tensor([float(rows)], device='cuda')
    rows_max = rows_all.clone()
    if world > 1:
        dist.all_reduce(rows_all)
        dist.all_reduce(rows_max, op=dist.ReduceOp.MAX)
    touched = int(((ends - starts) > 0).sum())
    flops = 2.0 * float(rows_all) * h * i * 3
    if nvfp4:
        l1_bytes = touched * (2 * i * h // 2 + 2 * i * h // 16) + rows * (h // 2 + h // 16) + rows * (i // 2 + i // 16)
        l2_bytes = touched * (h * i // 2 + h * i // 16) + rows * (i // 2 + i // 16) + rows * h * 2
    else:
        l1_bytes = touched * (2 * i * h // 2 + 2 * i * h // 32) + rows * (h + h // 32) + rows * (i + i // 32)
        l2_bytes = touched * (h * i // 2 + h * i // 32) + rows * (i + i // 32) + rows * h * 2
    times = torch.tensor([ms_per_step, e2e_ms] + stage_ms, dtype=torch.float64, device='cuda')
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_per_step, e2e_ms = float(times[0]), float(times[1])
    stage_ms = [float(v) for v in times[2:]]
    if rank != 0:
        return
    peak, peak_kind = measured_peaks()
    l1_gbs = l1_bytes / (stage_ms[2] * 1e-3) / 1e9
    tflops = flops / (ms_per_step * 1e-3) / 1e12
    line = {
        'metric': METRIC, 'value': t * world / (ms_per_step * 1e-3), 'unit': 'tokens/s', 'n_gpus': world,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms_per_step, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': cfg.get('mma', 'fp8xfp4') + ' (fp32 accumulate)', 'data': 'synthetic',
        'config': workload_config(cfg, world),
        'e2e': {'value': t * world / (e2e_ms * 1e-3), 'unit': 'tokens/s', 'ms_per_step': e2e_ms,
                'h2d_bytes_per_step': x_host.numel() * 2 + logits_host.numel() * 4, 'd2h_bytes_per_step': y_host.numel() * 2},
        'gpu_launches': kernels_per_step * args.steps,
        'clocks': clocks,
        # the gate/up GEMM is split by expert size over the two tile orientations: the timed stage holds both launches
        # and, for the swapped half, the small SwiGLU + requant kernel (single rank, FP8 kind; otherwise one launch)
        'roofline': {'kernel': 'gate/up GEMM + SwiGLU + FP8 requant (dgb200_grouped_gemm_kernel + dgb200_swap_gemm_kernel + '
                               'dgb200_swiglu_requant_rows_kernel)' if (world == 1 and not nvfp4) else
                               'dgb200_grouped_gemm_kernel (L1: gate/up GEMM + SwiGLU + requant)', 'bound': 'hbm',
                     'achieved': l1_gbs, 'peak': peak, 'unit': 'GB/s', 'frac': l1_gbs / peak, 'peak_source': peak_kind,
                     'traffic': int(L1_KERNEL_DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE * l1_bytes), 'algorithmic_bytes': l1_bytes, 'kernel_ms': stage_ms[2]},
        'stages_ms': {'plan': stage_ms[0], 'dispatch': stage_ms[1], 'l1_gemm_swiglu': stage_ms[2],
                      'l2_gemm': stage_ms[3], 'combine': stage_ms[4]},
        'l2_gemm_hbm_gbs': l2_bytes / (stage_ms[3] * 1e-3) / 1e9,
        'tflops': tflops,
        'frac_fp4_dense_peak_nominal': tflops / (FP4_DENSE_PEAK_TFLOPS_NOMINAL * world),
        'frac_fp8_rate_peak_nominal': tflops / (FP8_DENSE_PEAK_TFLOPS_NOMINAL * world),
        'routed_rows': rows,
        'load_imbalance_max_over_mean': float(rows_max) / (float(rows_all) / world) if float(rows_all) > 0 else None,
    }
    if world == 1 and not args.skip_cpu_baseline:
        idx, w = buf.topk_idx[:t].cpu(), buf.topk_weights[:t].cpu()
        from oracle import quant
        x_q_g, x_sf_g = dg.utils.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=32, use_packed_ue8m0=True)
        x_q_c, x_sf_c = x_q_g.cpu(), quant.unpack_ue8m0(x_sf_g.cpu())
        sample = dict(cpu_weights)
        sample.update({'x_q': [], 'x_sf': [], 'w': []})
        for g in range(CPU_SAMPLE_EXPERTS):
            tok, slot = torch.nonzero(idx == g, as_tuple=True)
            sample['x_q'].append(x_q_c[tok])
            sample['x_sf'].append(x_sf_c[tok])
            sample['w'].append(w[tok, slot])
        srows, dt, cores = time_cpu_sample(sample, 3, 1)
        line['cpu_baseline'] = {'value': srows / k / dt, 'unit': 'tokens/s', 'cores': cores, 'kind': 'port',
                                'sample': sample_description(cfg, srows)}
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
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
    run_ours(args, cfg, rank, world, local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
