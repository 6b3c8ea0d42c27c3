"""bench.py's clock samplers on CPU: the in-process NVML sampler against a fake NVML module (read-only queries only), and
the nvidia-smi sampler's parser with its cut to the timed region."""
import datetime
import sys
import time
import types

import bench


def test_nvml_sampler_reads_clocks_and_reasons(monkeypatch):
    import torch
    fake = types.ModuleType('pynvml')
    fake.NVML_CLOCK_SM = 1
    fake.nvmlInit = lambda: None
    fake.nvmlDeviceGetHandleByUUID = lambda uuid: ('handle', uuid)
    fake.nvmlDeviceGetHandleByIndex = lambda index: ('handle', index)
    fake.nvmlDeviceGetMaxClockInfo = lambda handle, kind: 1965
    fake.nvmlDeviceGetClockInfo = lambda handle, kind: 1410
    fake.nvmlDeviceGetCurrentClocksEventReasons = lambda handle: 0x4  # sw_power_cap
    monkeypatch.setitem(sys.modules, 'pynvml', fake)
    monkeypatch.setattr(torch.cuda, 'get_device_properties', lambda index: types.SimpleNamespace(uuid='0000'))
    sampler = bench.make_clock_sampler(0)
    assert isinstance(sampler, bench.NvmlClockSampler)
    sampler.start()
    time.sleep(0.02)  # not yet inside the timed region: nothing is recorded
    sampler.begin()
    time.sleep(0.05)
    sampler.end()
    got = sampler.stop()
    assert got['sm_mhz'] == 1410.0 and got['sm_max_mhz'] == 1965.0 and got['reasons'] == ['sw_power_cap']
    assert 3 <= got['samples'] <= 20 and got['source'] == 'nvml'


def test_sampler_falls_back_without_nvml(monkeypatch):
    monkeypatch.setitem(sys.modules, 'pynvml', None)  # import raises
    assert isinstance(bench.make_clock_sampler(0), bench.ClockSampler)


def test_nvidia_smi_samples_are_cut_to_the_timed_region():
    sampler = bench.ClockSampler(0)
    sampler.proc = types.SimpleNamespace(terminate=lambda: None, wait=lambda: None)
    now = datetime.datetime.now()
    for i in range(-10, 10):
        t = now + datetime.timedelta(milliseconds=20 * i)
        stamp = t.strftime('%Y/%m/%d %H:%M:%S.') + '%03d' % (t.microsecond // 1000)
        sampler.file.write(f'{stamp}, 0, {1500 + i}, 1965, 900.1, 0x4, Not Active, Not Active, Not Active, '
                           f'{"Active" if i == 0 else "Not Active"}\n')
    sampler.t_begin = now - datetime.timedelta(milliseconds=50)
    sampler.t_end = now + datetime.timedelta(milliseconds=50)
    got = sampler.stop()
    assert got['samples'] in (5, 6) and got['sm_mhz'] in (1500.0, 1501.0) and got['reasons'] == ['sw_power_cap']
    assert got['window'] == 'timed region'
