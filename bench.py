#!/usr/bin/env python
"""Benchmark of the hybrid-cache decode layer-step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config C]

One step = the new token's cache write for every request (K/V rows for K/V-cached
requests, the layer-input row for hidden-cached ones) followed by hybrid decode
attention over the whole ragged batch, through one native call
(``attention.decode_layer_step``).  With N > 1 the attention heads and the matching
W_k / W_v / W_o slices are sharded over the N ranks (hidden cache replicated) and the
step also holds the o_proj GEMM and its all-reduce: strong scaling, the batch is fixed.

The headline workload is configuration 2 (OPT-13B layer, fp16, 256 requests, lognormal
context lengths, half of them hidden-cached).  Prints ONE JSON line on rank 0.  After the
timed region the default run adds, each with its own clock sample:

  roofline_kv_path_pure / roofline_reprojection_pure   the K/V-only and the hidden-only
        sub-batch of configuration 2, each kernel running alone;
  roofline_cache_writes   configuration 3's prefill cache writes + block copies, alone and
        inside the loaded step;
  config5_sweep           configuration 5 at 0 / 25 / 50 / 75 / 100 % hidden-cached;
  config4                 configuration 4 (OPT-66B, bf16, 512 requests) at tp = N;
  tp_check (N > 1)        the all-reduced o_proj output of four requests against the
                          unsharded product formed on rank 0.

``--impl reference`` runs the reference's own op chain on the GPU (its CUDA source compiled
unmodified + the library kernels it calls, see oracle/literal_chain_gpu.py) on the same
configuration, seed and requests, and the CPU restatement of it beside it.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "hybrid-cache decode tokens/s @OPT-13B layer, B=256"
UNIT = "tokens/s"
TOL = "|x - ref| <= 2e-2 + 2e-2 * |ref|"


# --------------------------------------------------------------------------- #
# helpers
# --------------------------------------------------------------------------- #
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "tflops_burst": float(p["bf16_tflops"]),
                "tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0,
                "source": "fallback"}


class ClockSampler:
    """Samples SM clock, board power and the clock-event (throttle) reasons of one GPU for the life
    of the benchmark -- through NVML every 10 ms where the bindings import (read-only queries, the
    same counters nvidia-smi prints), else through one ``nvidia-smi -lms 100`` process;
    ``window(t0, t1)`` summarises the samples of a time window."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.samples = []        # (arrival time, sm MHz, max sm MHz, watts, set of reasons)
        self.thread = None
        self.stopping = False
        self.source = None

    # -- NVML ------------------------------------------------------------------------ #
    def _start_nvml(self):
        import pynvml
        pynvml.nvmlInit()
        handle = None
        try:
            uuid = str(torch.cuda.get_device_properties(self.gpu_index).uuid)
            handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
        reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons",
                             getattr(pynvml, "nvmlDeviceGetCurrentClocksThrottleReasons", None))
        bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        mx = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
        pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)   # fails here, not in the thread

        def pump():
            while not self.stopping:
                try:
                    mhz = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                    watts = pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0
                    mask = int(reasons_fn(handle)) if reasons_fn is not None else 0
                    self.samples.append((time.perf_counter(), mhz, mx, watts,
                                         {n for n, b in bits.items() if mask & b}))
                except Exception:
                    pass
                time.sleep(0.01)

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()
        self.source = "NVML, every 10 ms"

    # -- nvidia-smi -------------------------------------------------------------------- #
    def _start_smi(self):
        self.proc = subprocess.Popen(
            ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
             "-lms", "100", "-i", str(self.gpu_index)],
            stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, bufsize=1)

        def pump():
            for line in self.proc.stdout:
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    self.samples.append((time.perf_counter(), float(f[1]), float(f[2]), float(f[3]),
                                         {n for n, v in zip(self.NAMES, f[5:9]) if v.lower().startswith("active")}))
                except ValueError:
                    continue

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()
        self.source = "nvidia-smi -lms 100"

    def start(self):
        try:
            self._start_nvml()
        except Exception:
            try:
                self._start_smi()
            except OSError:
                self.source = None

    @property
    def lines(self):
        return self.samples

    def stop(self):
        self.stopping = True
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def window(self, t_begin: float, t_end: float, lead: float = 0.0):
        """Samples that arrived in ``[t_begin, t_end]``.  A window shorter than the sampling
        interval may hold none: then the samples of the ``lead`` seconds of identical load
        just before it are used and ``window`` says so."""
        if self.source is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source available"]}
        inside = [x for x in self.samples if t_begin <= x[0] <= t_end + 0.005]
        where = "timed region"
        if not inside and lead > 0:
            inside = [x for x in self.samples if t_begin - lead <= x[0] < t_begin]
            where = f"untimed steps of the same load in the {lead:.1f} s before the timed region (region shorter than the sampling interval)"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"], "source": self.source}
        sm = [x[1] for x in inside]
        power = [x[3] for x in inside]
        reasons = set().union(*[x[4] for x in inside])
        return {"sm_mhz": statistics.median(sm), "sm_min_mhz": min(sm), "sm_max_mhz": max(x[2] for x in inside),
                "reasons": sorted(reasons), "samples": len(sm), "power_w_max": round(max(power), 1),
                "power_w_median": round(statistics.median(power), 1), "window": where, "source": self.source}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), \
        int(os.environ.get("WORLD_SIZE", 1))


def dtype_name(dt):
    return {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}[dt]


def cpu_sample_requests(lens, hid, flop_budget, e, hd):
    """A bounded sample of the batch for the host-core baseline: hidden requests in
    batch order until their re-projection reaches ``flop_budget`` FLOPs, and as many
    K/V requests, which keeps the configuration's cache-type mix."""
    picked_h, flops = [], 0.0
    for r, (s, h) in enumerate(zip(lens, hid)):
        if h:
            picked_h.append(r)
            flops += 2.0 * s * e * 2 * hd
            if flops >= flop_budget:
                break
    n_h_total = sum(1 for h in hid if h)
    n_kv_total = len(hid) - n_h_total
    want_kv = len(picked_h) if n_h_total == 0 else round(len(picked_h) * n_kv_total / max(1, n_h_total))
    if not picked_h:
        want_kv = min(n_kv_total, 32)
    picked_kv = [r for r, h in enumerate(hid) if not h][:want_kv]
    return sorted(picked_h + picked_kv)


def run_cpu_port(workload_cpu, requests, steps, warmup):
    """The oracle's layer-step (cache writes + hybrid decode attention, fp32) on the host
    cores for the sampled requests; returns seconds per step."""
    from oracle import hybrid_cache_oracle as O
    w = workload_cpu
    wk, bk, wv, bv = w.kv_weights()
    wk, wv = wk.float(), wv.float()
    bk, bv = bk.float(), bv.float()

    def one():
        return O.decode_layer_step(w.hidden_states, w.query, w.new_key, w.new_value, w.kv_cache,
                                   w.hidden_cache, wk, bk, wv, bv, w.meta, w.scale,
                                   requests=requests)
    for _ in range(warmup):
        one()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    return (time.perf_counter() - t0) / max(1, steps)


def cpu_baseline_block(w, lens, hid, flop_budget, steps=2):
    shape = w.shape
    hd = w.heads * shape.head_dim
    sample = cpu_sample_requests(lens, hid, flop_budget, shape.hidden, hd)
    cpu_w = w.cpu()
    sec = run_cpu_port(cpu_w, sample, steps, 0)
    return {"value": round(len(sample) / sec, 3), "unit": UNIT, "cores": torch.get_num_threads(),
            "host_cpus": os.cpu_count(), "kind": "port",
            "sample": f"{len(sample)} of {len(lens)} requests in batch order keeping the hidden/K-V mix "
                      f"({sum(lens[r] for r in sample)} cached tokens), {steps} steps of "
                      f"{sec:.2f} s each; tokens/s = sampled requests / time"}


# --------------------------------------------------------------------------- #
# the step
# --------------------------------------------------------------------------- #
class LayerStep:
    """Holds one rank's tensors and runs the measured step through the package's public API."""

    def __init__(self, w, tp_group=None, tp_comm=None):
        from apt_serve_b200 import attention as A
        self.A = A
        self.w = w
        self.tp_group = tp_group
        self.tp_comm = tp_comm
        m = w.meta
        h, d = w.heads, w.shape.head_dim
        self.h, self.d = h, d
        self.wk, self.bk, self.wv, self.bv = w.kv_weights()
        self.out = torch.empty_like(w.query)
        self.prefill_events = None   # (start, stop) recorded around prefill_writes when set
        self.workspace = A.attention_workspace(w.query.device, w.query.shape[0],
                                               m.private_block_tables.shape[1], w.shape.block_size, h, d)

    def layer_step(self, query, hidden_states, new_key, new_value, tables, seq_lens, cache_type, out=None):
        """New-token cache writes + hybrid decode attention: one native call."""
        w = self.w
        return self.A.decode_layer_step(query, hidden_states, new_key, new_value, w.kv_cache, w.hidden_cache,
                                        self.wk, self.bk, self.wv, self.bv, tables, seq_lens, cache_type,
                                        w.scale, out=self.out if out is None else out, workspace=self.workspace)

    def o_proj(self, attn_out):
        import torch.distributed as dist
        y = torch.nn.functional.linear(attn_out, self.w.o_weight)
        if self.tp_comm is not None:
            self.tp_comm.all_reduce(y)          # aps_tp_allreduce: the library's NCCL communicator
        else:
            dist.all_reduce(y, group=self.tp_group)
        return y.add_(self.w.o_bias)

    def prefill_writes(self):
        """Configuration 3: cache the packed prompt tokens (K/V rows of K/V-designated
        prompts, layer-input rows of hidden-designated ones) and copy 5 % of the blocks."""
        from apt_serve_b200 import ops
        from apt_serve_b200.attention import FlashAttentionBackend
        w, pf = self.w, self.w.prefill
        pm = pf.meta
        ops.prefill_cache_write(pf.key, pf.value, pf.hidden_states, w.kv_cache, w.hidden_cache,
                                pm.slot_mapping, pm.kv_cache_use_tot, pm.hidden_cache_use_input)
        if w.copy_pairs is not None:
            FlashAttentionBackend.copy_blocks([w.kv_cache], w.copy_pairs)

    def prefill_write_bytes(self):
        """Algorithmic bytes of prefill_writes: read + write of every payload."""
        w, pf = self.w, self.w.prefill
        es = w.shape.es
        n_kv = pf.meta.kv_cache_use_tot.numel()
        n_h = pf.meta.hidden_cache_use_input.numel()
        row_kv = 2 * self.h * self.d * es
        total = 2 * (n_kv * row_kv + n_h * w.shape.hidden * es)
        if w.copy_pairs is not None:
            total += 2 * w.copy_pairs.shape[0] * 2 * w.shape.block_size * self.h * self.d * es
        return total

    def step(self):
        w, m = self.w, self.w.meta
        if w.prefill is not None:
            if self.prefill_events is not None:
                self.prefill_events[0].record()
            self.prefill_writes()
            if self.prefill_events is not None:
                self.prefill_events[1].record()
        out = self.layer_step(w.query, w.hidden_states, w.new_key, w.new_value, m.private_block_tables,
                              m.seq_lens_tensor, m.cache_type)
        if self.tp_group is not None:
            out = self.o_proj(out)
        return out

    def step_absorbed(self):
        """The same step with the hidden requests attended through absorbed projections
        (attention.hybrid_decode_attention_absorbed) instead of the re-projecting kernel."""
        from apt_serve_b200 import mixed_cache_ops, ops
        w, m = self.w, self.w.meta
        if not hasattr(self, "_kv_new_slots"):
            new_slot = m.slot_mapping[m.hidden_holder_upd]
            self._kv_new_slots = torch.where(m.cache_type != 0, torch.full_like(new_slot, -1), new_slot)
        ops.reshape_and_cache_flash(w.new_key.view(-1, self.h, self.d), w.new_value.view(-1, self.h, self.d),
                                    w.kv_cache[0], w.kv_cache[1], self._kv_new_slots, "auto")
        mixed_cache_ops.hidden_to_cache(w.hidden_states, w.hidden_cache, m.slot_mapping,
                                        m.hidden_cache_use_input, m.hidden_cache_store_tot)
        return self.A.hybrid_decode_attention_absorbed(
            w.query, w.kv_cache, w.hidden_cache, self.wk, self.bk, self.wv, self.bv, m.private_block_tables,
            m.seq_lens_tensor, m.cache_type, w.scale, hidden_rows=m.hidden_cache_use_input, out=self.out)


class Timer:
    """Device timing of K calls of ``fn`` with per-kernel events from the library's hook."""

    def __init__(self, dev, tp, sampler):
        self.dev, self.tp, self.sampler = dev, tp, sampler

    def barrier(self):
        torch.cuda.synchronize()
        if self.tp > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def run(self, fn, steps, warmup, preload_s=0.0, step_obj=None):
        """``warmup`` untimed calls, optionally ``preload_s`` seconds more of the same load (so that
        the power state has settled and clock samples exist), then ``steps`` timed calls.  Returns
        a dict with ms per step (max over ranks), per-kernel ms from the profile-event hook,
        the clock sample of the window and time x median SM MHz."""
        from apt_serve_b200 import _native as N
        lib = N.lib()
        self.barrier()
        t_w = time.perf_counter()
        for _ in range(max(warmup, 3)):
            fn()
        self.barrier()
        warm_step_s = (time.perf_counter() - t_w) / max(warmup, 3)
        if preload_s > 0:
            # chunks of ~50 ms until the sampler has delivered and preload_s has passed (3 s at
            # most); rank 0 decides so that every rank runs the same number of collectives
            chunk_t = torch.tensor([min(2000, max(1, int(0.05 / max(warm_step_s, 1e-5))))], device=self.dev)
            if self.tp > 1:
                torch.distributed.broadcast(chunk_t, src=0)
            chunk = int(chunk_t.item())
            t_pre = time.perf_counter()
            while True:
                for _ in range(chunk):
                    fn()
                torch.cuda.synchronize()
                waited = time.perf_counter() - t_pre
                have = self.sampler is None or bool(self.sampler.lines)
                go_on = torch.tensor([int((waited < preload_s or not have) and waited < 3.0)], device=self.dev)
                if self.tp > 1:
                    torch.distributed.broadcast(go_on, src=0)
                if not int(go_on.item()):
                    break
        ev = lambda: torch.cuda.Event(enable_timing=True)
        ev_kv = [(ev(), ev()) for _ in range(steps)]
        ev_hid = [(ev(), ev()) for _ in range(steps)]
        ev_pf = [(ev(), ev()) for _ in range(steps)]
        for a, b in ev_kv + ev_hid + ev_pf:   # create the underlying handles
            a.record(); b.record()
        self.barrier()
        t0 = time.perf_counter()
        e0, e1 = ev(), ev()
        e0.record()
        for i in range(steps):
            if step_obj is not None and step_obj.w.prefill is not None:
                step_obj.prefill_events = ev_pf[i]
            lib.aps_set_profile_events(0, ctypes.c_void_p(ev_kv[i][0].cuda_event), ctypes.c_void_p(ev_kv[i][1].cuda_event))
            lib.aps_set_profile_events(1, ctypes.c_void_p(ev_hid[i][0].cuda_event), ctypes.c_void_p(ev_hid[i][1].cuda_event))
            fn()
        e1.record()
        self.barrier()
        t1 = time.perf_counter()
        lib.aps_set_profile_events(0, None, None)
        lib.aps_set_profile_events(1, None, None)
        if step_obj is not None:
            step_obj.prefill_events = None
        t = torch.tensor([e0.elapsed_time(e1)], device=self.dev, dtype=torch.float64)
        if self.tp > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item()) / steps
        res = {"ms_per_step": ms,
               "kv_ms": statistics.mean(a.elapsed_time(b) for a, b in ev_kv),
               "hid_ms": statistics.mean(a.elapsed_time(b) for a, b in ev_hid),
               "pf_ms": (statistics.mean(a.elapsed_time(b) for a, b in ev_pf)
                         if step_obj is not None and step_obj.w.prefill is not None else None)}
        if self.sampler is not None:
            res["clocks"] = self.sampler.window(t0, t1, lead=max(preload_s, 0.3))
            mhz = res["clocks"].get("sm_mhz")
            res["ms_x_sm_mhz"] = round(ms * mhz, 1) if mhz else None
        return res


def kernel_rooflines(work, res, peaks):
    """The two attention kernels' roofline blocks from per-kernel event times."""
    hid_ms, kv_ms = res["hid_ms"], res["kv_ms"]
    tflops = work["reprojection_flops"] / (hid_ms * 1e-3) / 1e12 if hid_ms > 0 and work["t_hidden"] else 0.0
    kv_gbs = work["kv_attention_bytes"] / (kv_ms * 1e-3) / 1e9 if kv_ms > 0 and work["t_kv"] else 0.0
    hidden = {"kernel": "hidden_path_kernel (tcgen05 re-projection + softmax partials)",
              "bound": "tensor", "achieved": round(tflops, 2), "peak": peaks["tflops_sustained"],
              "unit": "TFLOP/s", "frac": round(tflops / peaks["tflops_sustained"], 4),
              "frac_of_burst_peak": round(tflops / peaks["tflops_burst"], 4),
              "peak_source": peaks["source"] + " (sustained bf16 figure: the kernel runs inside a long step)",
              "ms_per_launch": round(hid_ms, 4), "flops_per_launch": work["reprojection_flops"]}
    kv = {"kernel": "kv_attention_tma_kernel (K/V streaming)", "bound": "hbm",
          "achieved": round(kv_gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
          "frac": round(kv_gbs / peaks["hbm_gbs"], 4), "peak_source": peaks["source"],
          "ms_per_launch": round(kv_ms, 4), "bytes_per_launch": work["kv_attention_bytes"]}
    return hidden, kv


# --------------------------------------------------------------------------- #
# end to end through the public API with host buffers
# --------------------------------------------------------------------------- #
class EndToEnd:
    """Every step: ONE host-to-device copy of the step's inputs out of a pinned staging buffer
    (layer input, query, new K/V rows, block tables, sequence lengths, cache types), the step
    through the public API, one device-to-host copy of the result.  Two steps are in flight:
    step i + 1's inputs are copied on a side stream while step i computes, results leave on a
    third stream, and the host waits for step i - 1's result before it enqueues step i + 1."""

    def __init__(self, st: LayerStep, dev, tp, out_shape, out_dtype):
        w, m = st.w, st.w.meta
        self.st, self.dev, self.tp = st, dev, tp
        src = {"hidden_states": w.hidden_states, "query": w.query, "new_key": w.new_key,
               "new_value": w.new_value, "tables": m.private_block_tables, "seq_lens": m.seq_lens_tensor,
               "cache_type": m.cache_type}
        self.layout, off = {}, 0
        for k, v in src.items():
            n = v.numel() * v.element_size()
            self.layout[k] = (off, n, v.dtype, tuple(v.shape))
            off = (off + n + 255) // 256 * 256
        self.h2d_bytes = sum(n for _, n, _, _ in self.layout.values())
        self.host = torch.empty(off, dtype=torch.uint8).pin_memory()
        for k, v in src.items():
            o, n, _, _ = self.layout[k]
            self.host[o:o + n] = v.contiguous().view(torch.uint8).view(-1).cpu()
        self.slots = []
        for _ in range(2):
            buf = torch.empty(off, dtype=torch.uint8, device=dev)
            views = {k: buf[o:o + n].view(dt).view(shape) for k, (o, n, dt, shape) in self.layout.items()}
            self.slots.append({"buf": buf, "in": views, "out": torch.empty(out_shape, dtype=out_dtype).pin_memory(),
                               "attn": torch.empty_like(w.query),   # the slot's own attention output
                               "h2d": torch.cuda.Event(), "computed": torch.cuda.Event(), "d2h": torch.cuda.Event()})
        self.d2h_bytes = self.slots[0]["out"].numel() * self.slots[0]["out"].element_size()
        self.copy_stream = torch.cuda.Stream(device=dev)
        self.out_stream = torch.cuda.Stream(device=dev)

    def enqueue(self, i):
        s = self.slots[i & 1]
        main = torch.cuda.current_stream()
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(s["computed"])      # the slot's previous step has read its inputs
            s["buf"].copy_(self.host, non_blocking=True)     # one cudaMemcpyAsync
            s["h2d"].record(self.copy_stream)
        main.wait_event(s["h2d"])
        main.wait_event(s["d2h"])                            # the slot's previous result has left the device
        v = s["in"]
        out = self.st.layer_step(v["query"], v["hidden_states"], v["new_key"], v["new_value"], v["tables"],
                                 v["seq_lens"], v["cache_type"], out=s["attn"])
        if self.tp > 1:
            out = self.st.o_proj(out)
        s["computed"].record(main)
        with torch.cuda.stream(self.out_stream):
            self.out_stream.wait_event(s["computed"])
            s["out"].copy_(out, non_blocking=True)
            s["d2h"].record(self.out_stream)
        out.record_stream(self.out_stream)

    def run(self, steps, barrier):
        for s in self.slots:
            s["computed"].record()
            s["d2h"].record()
        for i in range(4):
            self.enqueue(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(steps):
            self.enqueue(i)
            if i > 0:
                self.slots[(i - 1) & 1]["d2h"].synchronize()   # the previous step's result is on the host
        self.slots[(steps - 1) & 1]["d2h"].synchronize()
        barrier()
        sec = (time.perf_counter() - t0) / steps
        self.last_result = self.slots[(steps - 1) & 1]["out"]
        t = torch.tensor([sec], device=self.dev, dtype=torch.float64)
        if self.tp > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())


# --------------------------------------------------------------------------- #
# our arm
# --------------------------------------------------------------------------- #
def tp_check(st: LayerStep, w, tp, rank, dev):
    """The all-reduced o_proj output of four sampled requests against the unsharded product
    formed on rank 0 from the all-gathered attention slices and W_o columns (fp32)."""
    import torch.distributed as dist
    m = w.meta
    attn = st.layer_step(w.query, w.hidden_states, w.new_key, w.new_value, m.private_block_tables,
                         m.seq_lens_tensor, m.cache_type).clone()
    y = st.o_proj(attn.clone())
    b = attn.shape[0]
    rows = sorted({0, b // 3, (2 * b) // 3, b - 1})
    idx = torch.tensor(rows, device=dev)
    a_loc = attn.index_select(0, idx).contiguous()
    a_all = [torch.empty_like(a_loc) for _ in range(tp)]
    w_all = [torch.empty_like(w.o_weight) for _ in range(tp)]
    dist.all_gather(a_all, a_loc)
    dist.all_gather(w_all, w.o_weight.contiguous())
    if rank != 0:
        return None
    a_full = torch.cat(a_all, dim=1).float()
    w_full = torch.cat(w_all, dim=1).float()
    ref = a_full @ w_full.t() + w.o_bias.float()
    got = y.index_select(0, idx).float()
    err = (got - ref).abs()
    bound = 2e-2 + 2e-2 * ref.abs()
    return {"requests": rows, "max_abs_err": round(float(err.max()), 6),
            "max_abs_ref": round(float(ref.abs().max()), 4), "tolerance": TOL,
            "ok": bool((err <= bound).all())}


def run_ours(args):
    from apt_serve_b200.workloads import (CONFIG_SHAPES, algorithmic_work, draw_decode_batch,
                                          draw_prefill_batch, make_decode_workload)
    rank, local_rank, world = dist_env()
    n_gpus = args.gpus
    assert world == n_gpus or world == 1, f"WORLD_SIZE {world} does not match --gpus {n_gpus}"
    tp = world
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    group = None
    if tp > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    tp_comm = None
    if tp > 1:
        # the exchange step through the C ABI (aps_tp_*); torch.distributed only carries the id
        from apt_serve_b200.tp_comm import TensorParallelComm
        tp_comm = TensorParallelComm.from_torch_distributed()
    peaks = measured_peaks()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler is not None:
        sampler.start()
    timer = Timer(dev, tp, sampler)
    K, W = args.steps, max(args.warmup, 3)
    extras = not args.no_extras

    def build(cfg, lens, hid, **kw):
        return make_decode_workload(CONFIG_SHAPES[cfg], lens, hid, 1000 + cfg, dev, tp_rank=rank, tp_size=tp, **kw)

    # ---- headline: configuration `cfg` (2 unless --config) ----
    cfg = args.config
    shape = CONFIG_SHAPES[cfg]
    seed = 1000 + cfg
    lens, hid = draw_decode_batch(cfg, seed, batch=args.batch, hidden_fraction=args.hidden_fraction)
    kw = {"prefill": draw_prefill_batch(), "copy_fraction": 0.05} if cfg == 3 else {}
    w = build(cfg, lens, hid, **kw)
    work = algorithmic_work(shape, lens, hid, tp)
    B = len(lens)
    st = LayerStep(w, group, tp_comm)
    check = tp_check(st, w, tp, rank, dev) if tp > 1 else None
    res = timer.run(st.step, K, W, preload_s=0.5, step_obj=st)
    ms_per_step = res["ms_per_step"]
    status = st.A.attention_status(st.workspace)
    roof_hidden, roof_kv = kernel_rooflines(work, res, peaks)
    if work["t_hidden"] > 0 and shape.dtype != torch.float32:
        roof_hidden.update(tensor_cycle_block(st, shape, lens, hid, tp))
    if shape.dtype == torch.float32:
        # fp32 runs the CUDA-core re-projection (tcgen05 has no fp32 MMA): the tensor peak is not its bound
        roof_hidden.update({"kernel": "hidden_simt_kernel (fp32 CUDA-core re-projection + softmax partials)",
                            "bound": "fp32 CUDA cores (no measured peak on file)", "peak": None, "frac": None,
                            "frac_of_burst_peak": None, "peak_source": None})
        roof_kv["kernel"] = "kv_attention_kernel (K/V streaming, CUDA-core arithmetic: fp32)"

    per_rank = per_rank_block(st, res, tp, dev, B, shape) if tp > 1 else None

    out_shape = (B, shape.hidden) if tp > 1 else tuple(w.query.shape)
    e2e = EndToEnd(st, dev, tp, out_shape, shape.dtype)
    e2e_s = e2e.run(K, timer.barrier)
    h2d_bytes, d2h_bytes = e2e.h2d_bytes, e2e.d2h_bytes
    # what arrived on the host is what the device-resident step computes from the same inputs
    e2e_diff = float((e2e.last_result.float() - st.step().float().cpu()).abs().max())
    status |= st.A.attention_status(st.workspace)

    line_extra = {}
    # ---- for information: the same step with absorbed projections (not the path the metric
    # is quoted on: the headline step re-projects on the tensor cores) ----
    if (extras and tp == 1 and work["t_hidden"] > 0 and st.A.absorbed_supported(w.heads, shape.hidden, shape.dtype)
            and shape.head_dim == 128 and w.prefill is None):
        ref_out = st.step().float().clone()
        out_abs = st.step_absorbed()
        diff = (out_abs.float() - ref_out).abs()
        outside = int((diff > 2e-2 + 2e-2 * ref_out.abs()).sum().item())
        r = timer.run(st.step_absorbed, K, 3)
        line_extra["absorbed_variant"] = {
            "ms_per_step": round(r["ms_per_step"], 4), "tokens_per_s": round(B / (r["ms_per_step"] * 1e-3), 2),
            "max_abs_diff_vs_headline_path": round(float(diff.max().item()), 6),
            "elements_outside_2e-2_tolerance": outside,
            "note": "opt-in variant (hybrid_decode_attention_absorbed): same result, scores and weighted sums "
                    "taken over the cached hidden rows directly; not the path the metric is quoted on"}

    # ---- the pure sub-batches of the headline configuration ----
    if extras and cfg in (2, 5) and tp == 1 and 0 < sum(hid) < B:
        m = w.meta
        for name, keep in (("roofline_kv_path_pure", [not h for h in hid]), ("roofline_reprojection_pure", list(hid))):
            rows = torch.tensor([r for r, k in enumerate(keep) if k], device=dev)
            sub = {"q": w.query.index_select(0, rows), "t": m.private_block_tables.index_select(0, rows),
                   "s": m.seq_lens_tensor.index_select(0, rows), "c": m.cache_type.index_select(0, rows)}
            sub_out = torch.empty_like(sub["q"])
            fn = lambda: st.A.hybrid_decode_attention(sub["q"], w.kv_cache, w.hidden_cache, st.wk, st.bk, st.wv,
                                                      st.bv, sub["t"], sub["s"], sub["c"], w.scale, out=sub_out,
                                                      workspace=st.workspace)
            r = timer.run(fn, K, 3, preload_s=0.3)
            sw = algorithmic_work(shape, [l for l, k in zip(lens, keep) if k], [h for h, k in zip(hid, keep) if k], tp)
            rh, rk = kernel_rooflines(sw, r, peaks)
            blk = rk if name == "roofline_kv_path_pure" else rh
            if name == "roofline_reprojection_pure":
                blk["traffic"] = None
            blk.update({"requests": int(rows.numel()), "call_ms": round(r["ms_per_step"], 4),
                        "clocks": r.get("clocks"), "kernel_ms_x_sm_mhz":
                            round(blk["ms_per_launch"] * r["clocks"]["sm_mhz"], 1)
                            if r.get("clocks") and r["clocks"].get("sm_mhz") else None,
                        "note": "the sub-batch of the headline configuration alone: no other kernel of the step runs"})
            line_extra[name] = blk
        status |= st.A.attention_status(st.workspace)

    # ---- a plain device copy in the position of the HBM-bound kernels, and the library GEMM the
    # tensor peak was measured with, on THIS box in THIS run ----
    if extras and cfg == 2 and tp == 1:
        line_extra["hbm_copy_yardstick"] = copy_yardstick(st, peaks, max(5, K // 2))
        line_extra["gemm_yardstick"] = gemm_yardstick(timer, peaks, roof_hidden)

    # ---- host-core baseline on a bounded sample (rank 0, N = 1 only) ----
    cpu_baseline = None
    if tp == 1 and not args.no_cpu_baseline:
        cpu_baseline = cpu_baseline_block(w, lens, hid, args.cpu_flops)

    pf_block = None
    if w.prefill is not None and res["pf_ms"]:
        pf_block = cache_write_block(st, res["pf_ms"], peaks, "inside the loaded step")
    del e2e, st, w
    torch.cuda.empty_cache()

    # ---- configuration 3: prefill cache writes + block copies ----
    if extras and cfg == 2 and tp == 1:
        l3, h3 = draw_decode_batch(3, 1003)
        w3 = build(3, l3, h3, prefill=draw_prefill_batch(), copy_fraction=0.05)
        st3 = LayerStep(w3)
        r_step = timer.run(st3.step, max(5, K // 2), 3, preload_s=0.4, step_obj=st3)
        blk = cache_write_block(st3, r_step["pf_ms"], peaks, "inside the loaded step (configuration 3: "
                                "prefill writes + block copies + decode step, back to back)")
        blk["clocks"] = r_step.get("clocks")
        blk["step_ms"] = round(r_step["ms_per_step"], 4)
        r_alone = timer.run(st3.prefill_writes, K, 3, preload_s=0.3)
        alone = cache_write_block(st3, r_alone["ms_per_step"], peaks, "the two launches alone, back to back")
        blk["alone"] = {k: alone[k] for k in ("ms_per_step", "achieved", "frac")}
        blk["alone"]["clocks"] = r_alone.get("clocks")
        line_extra["roofline_cache_writes"] = blk
        del st3, w3
        torch.cuda.empty_cache()
    elif pf_block is not None:
        line_extra["roofline_cache_writes"] = pf_block

    # ---- configuration 5: hidden fraction swept ----
    if extras and cfg == 2 and tp == 1:
        sweep = []
        for frac in (0.0, 0.25, 0.5, 0.75, 1.0):
            l5, h5 = draw_decode_batch(5, 1005, hidden_fraction=frac)
            w5 = build(5, l5, h5)
            st5 = LayerStep(w5)
            r = timer.run(st5.step, max(5, K // 2), 3, preload_s=0.3)
            wk5 = algorithmic_work(CONFIG_SHAPES[5], l5, h5, tp)
            rh, rk = kernel_rooflines(wk5, r, peaks)
            sweep.append({"hidden_fraction": frac, "ms_per_step": round(r["ms_per_step"], 4),
                          "tokens_per_s": round(len(l5) / (r["ms_per_step"] * 1e-3), 1),
                          "reprojection_tflops": rh["achieved"] if wk5["t_hidden"] else None,
                          "reprojection_frac": rh["frac"] if wk5["t_hidden"] else None,
                          "kv_path_gbs": rk["achieved"] if wk5["t_kv"] else None,
                          "kv_path_frac": rk["frac"] if wk5["t_kv"] else None,
                          "clocks": r.get("clocks"), "ms_x_sm_mhz": r.get("ms_x_sm_mhz")})
            status |= st5.A.attention_status(st5.workspace)
            del st5, w5
            torch.cuda.empty_cache()
        line_extra["config5_sweep"] = {"workload": "OPT-13B layer, fp16, 64 requests of 1536..2048 tokens", "points": sweep}

    # ---- configuration 4 at tp = N ----
    if extras and cfg == 2:
        l4, h4 = draw_decode_batch(4, 1004)
        w4 = build(4, l4, h4)
        st4 = LayerStep(w4, group, tp_comm)
        k4 = max(3, K // 4) if tp == 1 else K
        r = timer.run(st4.step, k4, 3, preload_s=0.4)
        wk4 = algorithmic_work(CONFIG_SHAPES[4], l4, h4, tp)
        rh, rk = kernel_rooflines(wk4, r, peaks)
        e4 = EndToEnd(st4, dev, tp, (len(l4), CONFIG_SHAPES[4].hidden) if tp > 1 else tuple(w4.query.shape),
                      CONFIG_SHAPES[4].dtype)
        e4_s = e4.run(k4, timer.barrier)
        status |= st4.A.attention_status(st4.workspace)
        line_extra["config4"] = {
            "workload": f"OPT-66B layer (72 heads x 128, hidden 9216), bf16, 512 decode requests, "
                        f"{sum(h4)} hidden-cached, tp = {tp} ({72 // tp} heads per rank)",
            "steps": k4, "ms_per_step": round(r["ms_per_step"], 4),
            "tokens_per_s": round(len(l4) / (r["ms_per_step"] * 1e-3), 1),
            "e2e_ms_per_step": round(e4_s * 1e3, 4), "e2e_tokens_per_s": round(len(l4) / e4_s, 1),
            "reprojection_ms": round(r["hid_ms"], 4), "reprojection_tflops_per_gpu": rh["achieved"],
            "kv_path_ms": round(r["kv_ms"], 4), "kv_path_gbs_per_gpu": rk["achieved"],
            "clocks": r.get("clocks"), "ms_x_sm_mhz": r.get("ms_x_sm_mhz")}
        del e4, st4, w4

    if tp_comm is not None:
        tp_comm.destroy()
    if sampler is not None:
        sampler.stop()
    if rank != 0:
        if tp > 1:
            torch.distributed.destroy_process_group()
        return

    roofline = dict(roof_hidden if work["t_hidden"] > 0 else roof_kv)
    # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum).  For the default workload
    # (configuration 2, one GPU, all 256 requests) they were captured on this very launch: the two
    # counters take one ncu pass, so nothing is saved or restored around the 5 GB the step holds.
    default_workload = cfg == 2 and tp == 1 and args.batch is None and args.hidden_fraction is None
    capture = ("`ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum --clock-control none -k regex:%s -s 3 -c 2 "
               "python bench.py --steps 2 --warmup 3 --no-cpu-baseline --no-extras` (1 pass per launch), two launches: ")
    if default_workload:
        roofline["traffic"] = 9_650_000_000
        roofline["traffic_source"] = (capture % "hidden_path" + "9.61 + 0.037 GB and 9.47 + 0.033 GB read + written, 8.9 x the "
                                      "mandatory bytes (hidden rows and W once: 1.08 GB): W and the hidden rows are re-streamed "
                                      "from HBM per round of work items, 1.2 TB/s = 18 % of the copy bandwidth; the figure moves "
                                      "with the GPU (7.4 - 7.6 GB, 9.3 - 10.5 GB and 13.0 GB on others for the same binary and "
                                      "inputs: the live set sits at the ~60 MB of L2 that serve data read from both dies), the "
                                      "kernel's time x clock does not")
        roof_kv["traffic"] = 2_040_000_000
        roof_kv["traffic_source"] = capture % "kv_attention_tma" + "2.02 + 0.02 GB, 1.02 x the algorithmic bytes"
    else:
        roofline["traffic"] = None
        roofline["traffic_source"] = ("not captured for this workload (captured for the default one: configuration 2, one GPU); "
                                      "the re-projection kernel's DRAM traffic depends on the work-order groups, not on the "
                                      "cached tokens alone, so it is not scaled from another case")
        roof_kv["traffic"] = int(1.02 * work["kv_attention_bytes"]) if work["t_kv"] else None
        roof_kv["traffic_source"] = ("1.02 x the algorithmic bytes, the ratio ncu measured on configuration 2 and on the "
                                     "16-request all-K/V case, scaled by the cached tokens")
    # the mixed step against its two lower bounds: every K/V byte at the measured copy bandwidth,
    # every re-projection FLOP at the measured sustained tensor rate; the step cannot beat the
    # larger of the two and would equal their sum if the two paths did not overlap at all
    t_kv = work["kv_attention_bytes"] / (peaks["hbm_gbs"] * 1e9) * 1e3 if work["t_kv"] else 0.0
    t_tc = work["reprojection_flops"] / (peaks["tflops_sustained"] * 1e12) * 1e3 if work["t_hidden"] else 0.0
    mixed = {"kv_bytes_at_copy_bandwidth_ms": round(t_kv, 4), "reprojection_flops_at_sustained_peak_ms": round(t_tc, 4),
             "step_ms": round(ms_per_step, 4),
             "frac_of_max_bound": round(max(t_kv, t_tc) / ms_per_step, 4),
             "frac_of_sum_bound": round((t_kv + t_tc) / ms_per_step, 4),
             "note": "lower bounds over the step's device time: max = the slower path alone, sum = both paths "
                     "back to back (they run back to back here: one stream, the re-projection kernel fills the SMs)"}
    launches = 5 + (2 if cfg == 3 else 0)
    line = {
        "metric": METRIC, "value": round(B / (ms_per_step * 1e-3), 2), "unit": UNIT, "n_gpus": n_gpus,
        "steps": K, "warmup": W, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": dtype_name(shape.dtype), "data": "synthetic",
        "config": {"workload": f"config {cfg}: {shape.name} layer ({shape.num_heads} heads x {shape.head_dim}, "
                               f"hidden {shape.hidden}), {B} decode requests, {sum(hid)} hidden-cached, seed {seed}",
                   "cached_tokens_per_rank_view": {"t_kv": work["t_kv"], "t_hidden": work["t_hidden"]},
                   "step": ("prefill cache writes + block copies + " if cfg == 3 else "") +
                           "new-token cache writes + hybrid decode attention" +
                           (" + o_proj + all-reduce" if tp > 1 else ""),
                   "parallelism": f"tp{tp}" if tp > 1 else "single GPU",
                   **({"all_reduce": "aps_tp_allreduce (NCCL)"} if tp > 1 else {}),
                   "l2": (f"inputs larger than L2: {(work['kv_attention_bytes'] + work['hidden_bytes']) / 1e9:.2f} GB streamed per step"
                          if work['kv_attention_bytes'] + work['hidden_bytes'] > 256e6 else
                          f"working set {(work['kv_attention_bytes'] + work['hidden_bytes']) / 1e6:.1f} MB fits in L2: the number is L2-warm"),
                   "seed": seed},
        "clocks": res.get("clocks"), "ms_x_sm_mhz": res.get("ms_x_sm_mhz"),
        "e2e": {"value": round(B / e2e_s, 2), "unit": UNIT, "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": d2h_bytes, "ms_per_step": round(e2e_s * 1e3, 4),
                "max_abs_diff_vs_device_resident_step": e2e_diff,
                "pipeline": "two steps in flight: one pinned staging buffer and one host-to-device copy per step on "
                            "a side stream, the step and the device-to-host copy of its result on the main stream; "
                            "the host waits for step i - 1's result before it enqueues step i + 1"},
        "gpu_launches": launches * K,
        "gpu_launches_per_step": {"count": launches,
                                  "kernels": "bulk_copy_kernel (new-token rows), plan_kernel, kv_attention_tma_kernel, "
                                             "hidden_path_kernel, combine_kernel" +
                                             (" + 2 bulk_copy_kernel launches of the prefill part" if cfg == 3 else "")},
        "roofline": roofline, "roofline_kv_path": roof_kv, "roofline_mixed_step": mixed,
        "device_status": status,
    }
    if check is not None:
        line["tp_check"] = check
    if per_rank is not None:
        line["per_rank"] = per_rank
    line.update(line_extra)
    if cpu_baseline is not None:
        line["cpu_baseline"] = cpu_baseline
    print(json.dumps(line))
    if tp > 1:
        torch.distributed.destroy_process_group()


def per_rank_block(st, res, tp, dev, batch, shape):
    """What every rank measured for its own two attention kernels in the timed region, the
    re-projection kernel's cycle count per rank, and the all-reduce of the step's [B, E] tensor
    timed alone (20 back-to-back calls): the step is as long as its slowest rank plus the
    exchange, and the ranks' GPUs do not sit at the same clock under the power cap."""
    import torch.distributed as dist
    mine = torch.tensor([res["hid_ms"], res["kv_ms"], float(st.A.reprojection_cycles(st.workspace))],
                        device=dev, dtype=torch.float64)
    allr = [torch.empty_like(mine) for _ in range(tp)]
    dist.all_gather(allr, mine)
    y = torch.zeros(batch, shape.hidden, device=dev, dtype=shape.dtype)
    reduce = (lambda: st.tp_comm.all_reduce(y)) if st.tp_comm is not None else (lambda: dist.all_reduce(y, group=st.tp_group))
    for _ in range(5):
        reduce()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        reduce()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / 20], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"reprojection_ms": [round(float(x[0]), 4) for x in allr],
            "kv_path_ms": [round(float(x[1]), 4) for x in allr],
            "reprojection_sm_cycles_cta0": [int(x[2]) for x in allr],
            "all_reduce_alone_ms": round(float(t.item()), 4),
            "all_reduce_bytes": int(y.numel() * y.element_size())}


def tensor_cycle_block(st, shape, lens, hid, tp):
    """The re-projection kernel's own cycle count (CTA 0, last launch) against the cycles the
    tensor cores need for its tiles: a pair of 128-row tiles x 128 K + 128 V columns costs
    512 SM cycles per 64-element slab of the hidden size (four M256 N256 K16 instructions), the
    74 CTA pairs take the tile pairs x heads round robin.  A utilisation figure that does not
    depend on a sampled clock."""
    sms = torch.cuda.get_device_properties(st.w.query.device).multi_processor_count
    subs = sum((s + 15) // 16 for s, h in zip(lens, hid) if h)      # 16-row blocks, packed 8 per tile
    tiles = (subs + 7) // 8
    units = (tiles + 1) // 2
    items = units * (shape.num_heads // tp) * shape.head_dim // 128
    rounds = -(-items // (sms // 2))
    need = rounds * (-(-shape.hidden // 64)) * 512
    cycles = st.A.reprojection_cycles(st.workspace)
    return {"sm_cycles_cta0": cycles, "tensor_bound_cycles": need,
            "tensor_cycle_fraction": round(need / cycles, 4) if cycles else None,
            "work_items_per_cta_pair": round(items / (sms // 2), 2)}


def gemm_yardstick(timer, peaks, roof_hidden):
    """The measured tensor peak is `torch.matmul` on 8192^3 bf16 (cuBLAS) in a seconds-long loop
    on one B200 of the pool; the power cap makes that figure move with the box.  The same GEMM
    (fp16, like the step) run here as a loaded loop, so that the re-projection kernel's TFLOP/s
    can be read against what the library reaches on this box in this run."""
    n = 8192
    dev = torch.device("cuda", torch.cuda.current_device())
    a = torch.randn(n, n, device=dev, dtype=torch.float16)
    b = torch.randn(n, n, device=dev, dtype=torch.float16)
    c = torch.empty(n, n, device=dev, dtype=torch.float16)
    r = timer.run(lambda: torch.matmul(a, b, out=c), 60, 5, preload_s=0.5)
    tflops = 2 * n ** 3 / (r["ms_per_step"] * 1e-3) / 1e12
    out = {"what": "torch.matmul 8192 x 8192 x 8192 fp16 (cuBLAS, yardstick only), 60 back-to-back calls after "
                   "half a second of the same", "tflops": round(tflops, 1), "ms_per_call": round(r["ms_per_step"], 4),
           "measured_sustained_peak": peaks["tflops_sustained"], "clocks": r.get("clocks")}
    if roof_hidden.get("achieved"):
        out["reprojection_kernel_over_this_gemm"] = round(roof_hidden["achieved"] / tflops, 4)
    return out


def copy_yardstick(st, peaks, steps):
    """`Tensor.copy_` (the kind of copy the measured HBM peak was taken with) timed alone and
    right behind the loaded decode step, where the K/V streaming and cache-write kernels run,
    at two sizes: about the bytes configuration 3's cache writes move (2 x 480 MiB) and about
    the bytes configuration 2's K/V path streams (2 x 1 GiB).  What a plain copy of that size
    reaches at the step's power-capped clocks."""
    dev = st.w.query.device
    src = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    dst = torch.empty_like(src)

    def timed(n, with_step):
        a, b = src[:n], dst[:n]
        for _ in range(3):
            if with_step:
                st.step()
            b.copy_(a)
        t_end = time.perf_counter() + 0.3
        while with_step and time.perf_counter() < t_end:
            st.step()
            torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for e0, e1 in evs:
            if with_step:
                st.step()
            e0.record()
            b.copy_(a)
            e1.record()
        torch.cuda.synchronize()
        ms = sorted(e0.elapsed_time(e1) for e0, e1 in evs)[len(evs) // 2]
        return round(2 * n / (ms * 1e-3) / 1e9, 1)

    out = {"what": "torch copy_ (library copy, yardstick only), read + write bytes, median of "
                   f"{steps}: alone, and enqueued right behind each loaded decode step", "peak": peaks["hbm_gbs"]}
    for name, n in (("480_MiB", 480 << 20), ("1_GiB", 1 << 30)):
        alone, behind = timed(n, False), timed(n, True)
        out[name] = {"alone_gbs": alone, "behind_the_step_gbs": behind,
                     "alone_frac": round(alone / peaks["hbm_gbs"], 4),
                     "behind_the_step_frac": round(behind / peaks["hbm_gbs"], 4)}
    return out


def cache_write_block(st, ms, peaks, where):
    nbytes = st.prefill_write_bytes()
    gbs = nbytes / (ms * 1e-3) / 1e9
    w = st.w
    return {"kernels": "bulk_copy_kernel x 2: prefill_cache_write (K/V rows + layer-input rows of the packed prompts) + copy_blocks (prefill part of configuration 3)",
            "bound": "hbm", "bytes_per_step": nbytes, "ms_per_step": round(ms, 4), "achieved": round(gbs, 1),
            "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4),
            "prefill_tokens": int(w.prefill.meta.num_prefill_tokens),
            "copied_blocks": 0 if w.copy_pairs is None else int(w.copy_pairs.shape[0]), "measured": where}


# --------------------------------------------------------------------------- #
# reference arm
# --------------------------------------------------------------------------- #
def run_reference(args):
    """The reference's decode op chain for the same configuration, seed and requests.

    On the GPU: the reference's own ``mixed_cache.cu`` (compiled unmodified, oracle/_ref) for
    hidden_to_cache / cache_to_hidden / mixed_kv_to_cache, ``F.linear`` for the kv_only
    projection, vLLM's flash-attention paged decode over the shared cache -- the kernels of
    aptserve_opt.py:106-124 and aptserve_flash_attn.py:356-387, 462-473 (the unmodified vLLM
    0.5.0.post1 engine around them cannot be installed here).  Beside it, as ``cpu_baseline``,
    the CPU restatement of the same path on the host cores on a bounded sample.  When a piece
    of the GPU chain is missing the line's value is the CPU figure and says so."""
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    torch.set_num_threads(max(1, os.cpu_count() or 1))   # torchrun exports OMP_NUM_THREADS=1 to its ranks
    from apt_serve_b200.workloads import CONFIG_SHAPES, draw_decode_batch, make_decode_workload
    cfg = args.config
    shape = CONFIG_SHAPES[cfg]
    seed = 1000 + cfg
    lens, hid = draw_decode_batch(cfg, seed, batch=args.batch, hidden_fraction=args.hidden_fraction)
    B = len(lens)
    K, W = args.steps, max(1, min(args.warmup, 3))
    gpu = None
    why = None
    if torch.cuda.is_available() and shape.dtype != torch.bfloat16:
        from oracle.literal_chain_gpu import LiteralChain
        chain, why = LiteralChain.create()
    else:
        chain = None
        why = "no CUDA device" if not torch.cuda.is_available() else "the reference's extension has no bf16 dispatch"
    if chain is not None:
        torch.cuda.set_device(local_rank)
        dev = torch.device("cuda", local_rank)
        w = make_decode_workload(shape, lens, hid, seed, dev, with_shared_cache=True)
        m = w.meta
        hd = w.heads * shape.head_dim
        w_kv, b_kv = w.qkv_weight[hd:], w.qkv_bias[hd:]

        def step(hidden_states, query, meta):
            return chain.hybrid_decode_layer(hidden_states, query, w_kv, b_kv, w.kv_cache, w.shared_cache, meta, w.scale)
        for _ in range(W):
            step(w.hidden_states, w.query, m)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            step(w.hidden_states, w.query, m)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / K
        # end to end: the step's inputs as the reference's model runner ships them every step
        # (layer input, query and the index tensors of the batch), result copied back
        names = ["slot_mapping", "slot_mapping_shared", "hidden_cache_use_tot", "kv_cache_use_tot",
                 "hidden_cache_use_input", "hidden_cache_store_tot", "hidden_holder_upd", "hidden_holder_pull",
                 "block_tables", "seq_lens_tensor"]
        host = {n: getattr(m, n).cpu().pin_memory() for n in names}
        host["hidden_states"] = w.hidden_states.cpu().pin_memory()
        host["query"] = w.query.cpu().pin_memory()
        devbuf = {n: torch.empty_like(v, device=dev) for n, v in host.items()}
        from dataclasses import replace
        m_dev = replace(m, **{n: devbuf[n] for n in names})
        host_out = torch.empty(tuple(w.query.shape), dtype=shape.dtype).pin_memory()

        def e2e_step():
            for n, v in host.items():
                devbuf[n].copy_(v, non_blocking=True)
            out = step(devbuf["hidden_states"], devbuf["query"], m_dev)
            host_out.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        for _ in range(2):
            e2e_step()
        t0 = time.perf_counter()
        for _ in range(K):
            e2e_step()
        e2e_s = (time.perf_counter() - t0) / K
        n_hid_tok, n_kv = int(m.slot_mapping_shared.numel()), int(m.kv_cache_use_tot.numel())
        gpu = {"ms": ms, "e2e_s": e2e_s,
               "h2d": sum(v.numel() * v.element_size() for v in host.values()),
               "d2h": host_out.numel() * host_out.element_size(),
               "attention": chain.attention_name,
               "notes": ([] if chain.inside_mixed_envelope(m) else
                         [f"mixed_kv_to_cache runs unmodified: with {n_hid_tok} cached hidden tokens and {n_kv} K/V "
                          "requests its hidden-token index (blockIdx.x % (2 * n_kv), mixed_cache.cu:88) aliases, so it "
                          "writes fewer distinct rows than intended (less traffic than the intended op; its output "
                          "is not checked here)"]) +
                        ["K/V-cached requests attend over the shared cache through their private ids, as the "
                         "reference does (aptserve_flash_attn.py:464-473)"]}
        del w
        torch.cuda.empty_cache()

    # the CPU restatement on a bounded sample of the same batch
    hd_full = shape.num_heads * shape.head_dim
    budget = min(args.cpu_flops, 6e13 / max(1, K)) if gpu is not None else min(args.cpu_flops, 2.4e14 / max(1, K))
    sample = cpu_sample_requests(lens, hid, budget, shape.hidden, hd_full)
    s_lens, s_hid = [lens[r] for r in sample], [hid[r] for r in sample]
    wc = make_decode_workload(shape, s_lens, s_hid, seed, "cpu")
    cpu_steps = K if gpu is None else min(K, 2)
    sec = run_cpu_port(wc, list(range(len(sample))), cpu_steps, min(args.warmup, 1) if gpu is None else 0)
    cpu_value = len(sample) / sec
    cpu_block = {"value": round(cpu_value, 3), "unit": UNIT, "cores": torch.get_num_threads(),
                 "host_cpus": os.cpu_count(), "kind": "port",
                 "sample": f"{len(sample)} of {B} requests of config {cfg} keeping the hidden/K-V mix "
                           f"({sum(s_lens)} cached tokens), {cpu_steps} steps of {sec:.2f} s; "
                           "tokens/s = sampled requests / time"}
    base = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": args.gpus, "steps": K,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "data": "synthetic",
            "cpu_baseline": cpu_block}
    wl = (f"config {cfg}: {shape.name} layer ({shape.num_heads} heads x {shape.head_dim}, hidden {shape.hidden}), "
          f"{B} decode requests, {sum(hid)} hidden-cached, seed {seed}")
    if gpu is not None:
        line = dict(base, value=round(B / (gpu["ms"] * 1e-3), 2), warmup=W, ms_per_step=round(gpu["ms"], 4),
                    dtype=dtype_name(shape.dtype),
                    config={"workload": wl, "seed": seed, "parallelism": "single GPU (rank 0)",
                            "step": "hidden_to_cache + zero-filled hidden_holder + cache_to_hidden + kv_only projection "
                                    "+ mixed_kv_to_cache + paged decode attention over the shared cache"},
                    reference_kernels={"kind": "reference",
                                       "mixed_cache_ops": "the reference's mixed_cache.cu compiled unmodified for sm_100a (oracle/_ref)",
                                       "projection": "torch.nn.functional.linear (cuBLAS)",
                                       "attention": gpu["attention"], "notes": gpu["notes"]},
                    e2e={"value": round(B / gpu["e2e_s"], 2), "unit": UNIT, "h2d_bytes_per_step": gpu["h2d"],
                         "d2h_bytes_per_step": gpu["d2h"], "ms_per_step": round(gpu["e2e_s"] * 1e3, 4)})
    else:
        line = dict(base, value=round(cpu_value, 3), warmup=min(args.warmup, 1), ms_per_step=round(sec * 1e3, 3),
                    dtype="f32",
                    config={"workload": wl + ", bounded sample on the host cores", "seed": seed},
                    reference_kernels={"kind": "port", "gpu_chain_unavailable": why},
                    e2e={"value": round(cpu_value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[1, 2, 3, 4, 5])
    ap.add_argument("--hidden-fraction", type=float, default=None)
    ap.add_argument("--batch", type=int, default=None, help="override the configuration's request count")
    ap.add_argument("--cpu-flops", type=float, default=2e13,
                    help="re-projection FLOPs of the host-core baseline's sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="headline measurement only (no sub-batch, configuration 3/4/5 blocks)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
