"""Sampled VRAM of this process while it generates, in the manner of `--vram-metrics`.

crates/metrics/src/memory.rs:11-64 (a footprint sampled every 100 ms, not an allocator's
high-water mark; start, peak, end and peak - start; a failed sample is kept as evidence even
if later ones succeed) and :119-138 (the `inference_vram_metrics {...}` line on stderr with
`request_id`, `model`, `status`, `error` and the snapshot's fields beside them).  The
reference asks NVML for the process's memory on the device with the CUDA context's UUID
(memory/nvml.rs:53-56); here NVML is asked the same through `pynvml`, and where the process
does not appear in its list (another PID namespace) or NVML cannot be loaded, the device's
used memory from the CUDA runtime stands in, and `vram_scope` says which it was.
"""
from __future__ import annotations

import json
import os
import sys
import threading
from typing import Callable, Optional, Tuple

SAMPLE_INTERVAL_MS = 100


class VramSampler:
    """`sample()` returns bytes or raises; it is called once at `start`, every `interval_ms` on a thread of its own, and once at `finish`."""

    def __init__(self, sample: Callable[[], int], scope: str, device_uuid: Optional[str], interval_ms: int = SAMPLE_INTERVAL_MS):
        self._sample, self._interval = sample, interval_ms / 1e3
        self.snapshot = {
            "vram_start_bytes": None, "vram_peak_sampled_bytes": None, "vram_end_bytes": None, "vram_peak_delta_bytes": None,
            "vram_sample_interval_ms": interval_ms, "vram_samples": 0, "vram_scope": scope, "vram_device_uuid": device_uuid,
            "vram_error": None,
        }
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def _observe(self) -> Optional[int]:
        try:
            value = int(self._sample())
        except Exception as error:  # a failed sample is recorded, never raised into the generation
            self.snapshot["vram_error"] = str(error)
            return None
        self.snapshot["vram_peak_sampled_bytes"] = max(self.snapshot["vram_peak_sampled_bytes"] or 0, value)
        self.snapshot["vram_samples"] += 1
        return value

    def start(self) -> "VramSampler":
        self.snapshot["vram_start_bytes"] = self._observe()

        def run():
            while not self._stop.wait(self._interval):
                self._observe()

        self._thread = threading.Thread(target=run, name="vram-sampler", daemon=True)
        self._thread.start()
        return self

    def finish(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        self.snapshot["vram_end_bytes"] = self._observe()
        peak, start = self.snapshot["vram_peak_sampled_bytes"], self.snapshot["vram_start_bytes"]
        if peak is not None and start is not None:
            self.snapshot["vram_peak_delta_bytes"] = max(0, peak - start)
        return self.snapshot


def report(snapshot: dict, model: str, request_id: int = 0, error: Optional[str] = None, stream=None) -> str:
    line = "inference_vram_metrics " + json.dumps(dict(
        {"request_id": request_id, "model": model, "status": "error" if error else "ok", "error": error}, **snapshot))
    print(line, file=stream or sys.stderr)
    return line


def device_sampler(device_index: int = 0) -> VramSampler:
    """A sampler of this process's memory on the CUDA device, or of the device's used memory where the process cannot be told apart."""
    import torch

    properties = torch.cuda.get_device_properties(device_index)
    uuid = getattr(properties, "uuid", None)
    uuid = None if uuid is None else "GPU-" + str(uuid)
    sample, scope = _process_sample(uuid)
    if sample is None:
        def sample():
            free, total = torch.cuda.mem_get_info(device_index)
            return total - free

        scope = "device"
    return VramSampler(sample, scope, uuid)


def _process_sample(uuid: Optional[str]) -> Tuple[Optional[Callable[[], int]], str]:
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode()) if uuid else pynvml.nvmlDeviceGetHandleByIndex(0)
        pid = os.getpid()

        def sample():
            for process in pynvml.nvmlDeviceGetComputeRunningProcesses(handle):
                if process.pid == pid and process.usedGpuMemory is not None:
                    return process.usedGpuMemory
            raise RuntimeError("this process is not in NVML's list for the device")

        sample()   # the process has a context by now; if it cannot be found once, it never will be
        return sample, "process_on_device"
    except Exception:
        return None, "device"
