#!/usr/bin/env python
"""Benchmark of the hybrid-cache decode layer-step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config C]

One step = the new token's cache write for every request (K/V rows for K/V-cached
requests, the layer-input row for hidden-cached ones) followed by hybrid decode
attention over the whole ragged batch.  With N > 1 the attention heads and the
matching W_k / W_v / W_o slices are sharded over the N ranks (hidden cache
replicated) and the step also holds the o_proj GEMM and its all-reduce.

N = 1 runs configuration 2 (OPT-13B layer, fp16, 256 requests, lognormal context
lengths, half of them hidden-cached).  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
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


# ncu, 16-request OPT-13B case (profiles/hidden_path_kernel_config5_b16_all_hidden.md,
# profiles/kv_attention_kernel_config5_b16_all_kv.md): dram read + write bytes per launch over the
# cached tokens of the launch
HIDDEN_DRAM_BYTES_PER_TOKEN = (3.007744e9 + 17.6e6) / 29088
KV_DRAM_BYTES_PER_TOKEN = (595.9e6 + 6.6e6) / 29088


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []          # (arrival time, text)
        self.reader = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, bufsize=1)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.lines.append((time.perf_counter(), line))

        self.reader = threading.Thread(target=pump, daemon=True)
        self.reader.start()

    def stop(self, t_begin: float, t_end: float):
        """Summary of the samples that arrived inside ``[t_begin, t_end]`` (the timed
        region).  A region shorter than the sampling interval may hold none: then the
        samples of the half second of identical load just before it are used, and
        ``window`` says so."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.reader.join(timeout=2)
        inside = [ln for t, ln in self.lines if t_begin <= t <= t_end + 0.02]
        window = "timed region"
        if not inside:
            inside = [ln for t, ln in self.lines if t_begin - 0.5 <= t < t_begin]
            window = "untimed steps of the same load in the 0.5 s before the timed region (region shorter than the sampling interval)"
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in inside:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power) if power else None, "window": window}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), \
        int(os.environ.get("WORLD_SIZE", 1))


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
        self.kv_rows = m.kv_request_rows
        self.kv_slots = m.slot_mapping[m.kv_cache_use_tot].contiguous()
        # per-request slot of the new token: K/V requests write K/V rows, hidden requests
        # write their layer-input row; the other kind is masked with -1 (skipped)
        new_slot = m.slot_mapping[m.hidden_holder_upd]
        self.kv_new_slots = torch.where(m.cache_type != 0, torch.full_like(new_slot, -1), new_slot)
        self.out = torch.empty_like(w.query)
        self.prefill_events = None   # (start, stop) recorded around prefill_writes when set
        self.fused_prefill_write = os.environ.get("APS_BENCH_FUSED_PREFILL_WRITE") is not None
        self.workspace = A.attention_workspace(w.query.device, w.query.shape[0],
                                               m.private_block_tables.shape[1], w.shape.block_size, h, d)

    def cache_writes(self, hidden_states, new_key, new_value, kv_new_slots):
        from apt_serve_b200 import mixed_cache_ops, ops
        w, m = self.w, self.w.meta
        ops.reshape_and_cache_flash(new_key.view(-1, self.h, self.d), new_value.view(-1, self.h, self.d),
                                    w.kv_cache[0], w.kv_cache[1], kv_new_slots, "auto")
        mixed_cache_ops.hidden_to_cache(hidden_states, w.hidden_cache, m.slot_mapping,
                                        m.hidden_cache_use_input, m.hidden_cache_store_tot)

    def attention(self, query, tables, seq_lens, cache_type):
        return self.A.hybrid_decode_attention(query, self.w.kv_cache, self.w.hidden_cache, self.wk,
                                              self.bk, self.wv, self.bv, tables, seq_lens, cache_type,
                                              self.w.scale, out=self.out, workspace=self.workspace)

    def o_proj(self, attn_out):
        import torch.distributed as dist
        y = torch.nn.functional.linear(attn_out, self.w.o_weight)
        if self.tp_comm is not None:
            self.tp_comm.all_reduce(y)          # aps_tp_allreduce: the library's NCCL communicator
        else:
            dist.all_reduce(y, group=self.tp_group)
        return y + self.w.o_bias

    def prefill_writes(self):
        """Configuration 3: cache the packed prompt tokens (K/V rows of K/V-designated
        prompts, layer-input rows of hidden-designated ones) and copy 5 % of the blocks."""
        from apt_serve_b200 import mixed_cache_ops, ops
        from apt_serve_b200.attention import FlashAttentionBackend
        w, pf = self.w, self.w.prefill
        pm = pf.meta
        if not hasattr(self, "_prefill_kv_slots"):
            slots = torch.full_like(pm.slot_mapping, -1)
            slots[pm.kv_cache_use_tot] = pm.slot_mapping[pm.kv_cache_use_tot]
            self._prefill_kv_slots = slots
        if self.fused_prefill_write:
            ops.prefill_cache_write(pf.key, pf.value, pf.hidden_states, w.kv_cache, w.hidden_cache,
                                    pm.slot_mapping, pm.kv_cache_use_tot, pm.hidden_cache_use_input)
        else:
            ops.reshape_and_cache_flash(pf.key, pf.value, w.kv_cache[0], w.kv_cache[1],
                                        self._prefill_kv_slots, "auto")
            mixed_cache_ops.hidden_to_cache(pf.hidden_states, w.hidden_cache, pm.slot_mapping,
                                            pm.hidden_cache_use_input, pm.hidden_cache_store_tot)
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
        self.cache_writes(w.hidden_states, w.new_key, w.new_value, self.kv_new_slots)
        out = self.attention(w.query, m.private_block_tables, m.seq_lens_tensor, m.cache_type)
        if self.tp_group is not None:
            out = self.o_proj(out)
        return out

    def step_absorbed(self):
        """The same step with the hidden requests attended through absorbed projections
        (attention.hybrid_decode_attention_absorbed) instead of the re-projecting kernel."""
        w, m = self.w, self.w.meta
        if w.prefill is not None:
            self.prefill_writes()
        self.cache_writes(w.hidden_states, w.new_key, w.new_value, self.kv_new_slots)
        out = self.A.hybrid_decode_attention_absorbed(
            w.query, w.kv_cache, w.hidden_cache, self.wk, self.bk, self.wv, self.bv, m.private_block_tables,
            m.seq_lens_tensor, m.cache_type, w.scale, hidden_rows=m.hidden_cache_use_input, out=self.out)
        if self.tp_group is not None:
            out = self.o_proj(out)
        return out


# --------------------------------------------------------------------------- #
# arms
# --------------------------------------------------------------------------- #
def run_ours(args):
    import ctypes
    from apt_serve_b200 import _native as N
    from apt_serve_b200.workloads import (CONFIG_SHAPES, algorithmic_work, draw_decode_batch,
                                          make_decode_workload)
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

    cfg = args.config
    shape = CONFIG_SHAPES[cfg]
    seed = 1000 + cfg
    lens, hid = draw_decode_batch(cfg, seed, batch=args.batch, hidden_fraction=args.hidden_fraction)
    extra = {}
    if cfg == 3:
        from apt_serve_b200.workloads import draw_prefill_batch
        extra = {"prefill": draw_prefill_batch(), "copy_fraction": 0.05}
    w = make_decode_workload(shape, lens, hid, seed, dev, tp_rank=rank, tp_size=tp, **extra)
    work = algorithmic_work(shape, lens, hid, tp)
    B = len(lens)
    tp_comm = None
    if tp > 1 and os.environ.get("APS_BENCH_TORCH_ALLREDUCE") is None:
        # the exchange step through the C ABI (aps_tp_*); torch.distributed only carries the id
        from apt_serve_b200.tp_comm import TensorParallelComm
        tp_comm = TensorParallelComm.from_torch_distributed()
    st = LayerStep(w, group, tp_comm)
    peaks = measured_peaks()

    def barrier():
        torch.cuda.synchronize()
        if tp > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: warm-up, then exactly K steps ----
    barrier()
    t_w = time.perf_counter()
    for _ in range(max(args.warmup, 3)):
        st.step()
    barrier()
    warm_step_s = (time.perf_counter() - t_w) / max(args.warmup, 3)
    K = args.steps
    ev_kv = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    ev_hid = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    for a, b in ev_kv + ev_hid:   # create the underlying handles
        a.record(); b.record()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # untimed steps of the same load while nvidia-smi comes up: chunks of ~50 ms until its first
    # sample has arrived and half a second has passed (3 s at most); rank 0 decides so that every
    # rank runs the same number of collectives
    chunk_t = torch.tensor([min(2000, max(1, int(0.05 / max(warm_step_s, 1e-5))))], device=dev)
    if tp > 1:
        torch.distributed.broadcast(chunk_t, src=0)
    chunk = int(chunk_t.item())
    t_pre = time.perf_counter()
    while True:
        for _ in range(chunk):
            st.step()
        torch.cuda.synchronize()
        waited = time.perf_counter() - t_pre
        go_on = torch.tensor([int((waited < 0.5 or not sampler.lines) and waited < 3.0)], device=dev)
        if tp > 1:
            torch.distributed.broadcast(go_on, src=0)
        if not int(go_on.item()):
            break
    barrier()
    t_region0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    lib = N.lib()
    ev_pf = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    e0.record()
    for i in range(K):
        st.prefill_events = ev_pf[i] if w.prefill is not None else None
        lib.aps_set_profile_events(0, ctypes.c_void_p(ev_kv[i][0].cuda_event), ctypes.c_void_p(ev_kv[i][1].cuda_event))
        lib.aps_set_profile_events(1, ctypes.c_void_p(ev_hid[i][0].cuda_event), ctypes.c_void_p(ev_hid[i][1].cuda_event))
        st.step()
    e1.record()
    barrier()
    t_region1 = time.perf_counter()
    st.prefill_events = None
    lib.aps_set_profile_events(0, None, None)
    lib.aps_set_profile_events(1, None, None)
    clocks = sampler.stop(t_region0, t_region1) if rank == 0 else None
    ms_total = e0.elapsed_time(e1)
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if tp > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms_per_step = float(t.item()) / K
    kv_ms = statistics.mean(a.elapsed_time(b) for a, b in ev_kv)
    hid_ms = statistics.mean(a.elapsed_time(b) for a, b in ev_hid)
    status = st.A.attention_status(st.workspace)
    pf_ms = statistics.mean(a.elapsed_time(b) for a, b in ev_pf) if w.prefill is not None else None

    # ---- end to end through the public API with host buffers ----
    m = w.meta
    host_in = {
        "hidden_states": w.hidden_states.cpu().pin_memory(), "query": w.query.cpu().pin_memory(),
        "new_key": w.new_key.cpu().pin_memory(), "new_value": w.new_value.cpu().pin_memory(),
        "tables": m.private_block_tables.cpu().pin_memory(), "seq_lens": m.seq_lens_tensor.cpu().pin_memory(),
        "cache_type": m.cache_type.cpu().pin_memory(), "kv_new_slots": st.kv_new_slots.cpu().pin_memory(),
    }
    dev_in = {k: torch.empty_like(v, device=dev) for k, v in host_in.items()}
    out_shape = (B, shape.hidden) if tp > 1 else tuple(w.query.shape)
    host_out = torch.empty(out_shape, dtype=shape.dtype).pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in host_in.values())
    d2h = host_out.numel() * host_out.element_size()

    def e2e_step():
        for k, v in host_in.items():
            dev_in[k].copy_(v, non_blocking=True)
        st.cache_writes(dev_in["hidden_states"], dev_in["new_key"], dev_in["new_value"], dev_in["kv_new_slots"])
        out = st.attention(dev_in["query"], dev_in["tables"], dev_in["seq_lens"], dev_in["cache_type"])
        if tp > 1:
            out = st.o_proj(out)
        host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / K
    t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
    if tp > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    e2e_s = float(t.item())

    # ---- for information: the same step with absorbed projections (not the path the metric
    # is quoted on: the headline step re-projects on the tensor cores) ----
    absorbed = None
    if (tp == 1 and work["t_hidden"] > 0 and shape.dtype in (torch.float16, torch.bfloat16)
            and shape.hidden % 512 == 0 and shape.head_dim == 128):
        ref_out = st.step().float().clone()
        for _ in range(3):
            out_abs = st.step_absorbed()
        diff = (out_abs.float() - ref_out).abs()
        outside = int((diff > 2e-2 + 2e-2 * ref_out.abs()).sum().item())
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a0.record()
        for _ in range(K):
            st.step_absorbed()
        a1.record()
        torch.cuda.synchronize()
        abs_ms = a0.elapsed_time(a1) / K
        absorbed = {"ms_per_step": round(abs_ms, 4), "tokens_per_s": round(B / (abs_ms * 1e-3), 2),
                    "max_abs_diff_vs_headline_path": round(float(diff.max().item()), 6),
                    "elements_outside_2e-2_tolerance": outside,
                    "note": "opt-in variant (hybrid_decode_attention_absorbed): same result, scores and "
                            "weighted sums taken over the cached hidden rows directly"}

    if tp_comm is not None:
        tp_comm.destroy()
    if rank != 0:
        if tp > 1:
            torch.distributed.destroy_process_group()
        return

    # DRAM bytes per launch, from the ncu captures summarised under profiles/ (16-request case of
    # the same OPT-13B shapes), scaled by the cached tokens a launch processes: both kernels'
    # traffic grows in proportion to them (hidden rows once plus the W rows re-streamed per
    # 16-tile group; K/V rows once).  Other shapes: not captured.
    opt13b = shape.name == "opt-13b" and tp == 1
    hid_traffic = int(HIDDEN_DRAM_BYTES_PER_TOKEN * work["t_hidden"]) if opt13b else None
    kv_traffic = int(KV_DRAM_BYTES_PER_TOKEN * work["t_kv"]) if opt13b else None
    tflops = work["reprojection_flops"] / (hid_ms * 1e-3) / 1e12 if hid_ms > 0 and work["t_hidden"] else 0.0
    kv_gbs = work["kv_attention_bytes"] / (kv_ms * 1e-3) / 1e9 if kv_ms > 0 and work["t_kv"] else 0.0
    if work["t_hidden"] > 0:
        roofline = {"kernel": "hidden_path_kernel (tcgen05 re-projection + softmax partials)",
                    "bound": "tensor", "achieved": round(tflops, 2), "peak": peaks["tflops_sustained"],
                    "unit": "TFLOP/s", "frac": round(tflops / peaks["tflops_sustained"], 4),
                    "frac_of_burst_peak": round(tflops / peaks["tflops_burst"], 4),
                    "peak_source": peaks["source"] + " (sustained bf16 figure: the kernel runs inside a long step)",
                    "ms_per_launch": round(hid_ms, 4), "flops_per_launch": work["reprojection_flops"],
                    "traffic": hid_traffic}
    else:
        roofline = {"kernel": "kv_attention_kernel", "bound": "hbm", "achieved": round(kv_gbs, 1),
                    "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(kv_gbs / peaks["hbm_gbs"], 4),
                    "peak_source": peaks["source"], "ms_per_launch": round(kv_ms, 4),
                    "bytes_per_launch": work["kv_attention_bytes"], "traffic": kv_traffic}
    roofline_kv = {"kernel": "kv_attention_kernel (K/V streaming)", "bound": "hbm",
                   "achieved": round(kv_gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                   "frac": round(kv_gbs / peaks["hbm_gbs"], 4), "ms_per_launch": round(kv_ms, 4),
                   "bytes_per_launch": work["kv_attention_bytes"], "traffic": kv_traffic}

    # ---- host-core baseline on a bounded sample (rank 0, N = 1 only) ----
    cpu_baseline = None
    if tp == 1 and not args.no_cpu_baseline:
        hd = w.heads * shape.head_dim
        sample = cpu_sample_requests(lens, hid, args.cpu_flops, shape.hidden, hd)
        cpu_w = w.cpu()
        sec = run_cpu_port(cpu_w, sample, 2, 0)
        cpu_baseline = {"value": round(len(sample) / sec, 3), "unit": UNIT, "cores": torch.get_num_threads(),
                        "host_cpus": os.cpu_count(), "kind": "port",
                        "sample": f"{len(sample)} of {B} requests in batch order keeping the hidden/K-V mix "
                                  f"({sum(lens[r] for r in sample)} cached tokens), two steps of "
                                  f"{sec:.2f} s each; tokens/s = sampled requests / time"}
        del cpu_w

    line = {
        "metric": METRIC, "value": round(B / (ms_per_step * 1e-3), 2), "unit": UNIT, "n_gpus": n_gpus,
        "steps": K, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "strong" if tp > 1 else "weak", "vs_baseline": None,
        "dtype": {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}[shape.dtype],
        "data": "synthetic",
        "config": {"workload": f"config {cfg}: {shape.name} layer ({shape.num_heads} heads x {shape.head_dim}, "
                               f"hidden {shape.hidden}), {B} decode requests, {sum(hid)} hidden-cached, "
                               f"T_kv={work['t_kv']} T_hidden={work['t_hidden']} cached tokens per rank view",
                   "step": ("prefill cache writes + block copies + " if w.prefill is not None else "") +
                           "new-token cache writes + hybrid decode attention" +
                           (" + o_proj + all-reduce" if tp > 1 else ""),
                   "parallelism": f"tp{tp}" if tp > 1 else "single GPU",
                   **({"all_reduce": "aps_tp_allreduce (NCCL)" if tp_comm is not None else "torch.distributed (NCCL)"}
                      if tp > 1 else {}),
                   "l2": (f"inputs larger than L2: {(work['kv_attention_bytes'] + work['hidden_bytes']) / 1e9:.2f} GB streamed per step"
                          if work['kv_attention_bytes'] + work['hidden_bytes'] > 256e6 else
                          f"working set {(work['kv_attention_bytes'] + work['hidden_bytes']) / 1e6:.1f} MB fits in L2: the number is L2-warm"),
                   "seed": seed},
        "clocks": clocks,
        "e2e": {"value": round(B / e2e_s, 2), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_s * 1e3, 4)},
        "gpu_launches": (6 + (3 if w.prefill is not None else 0)) * K,
        "roofline": roofline, "roofline_kv_path": roofline_kv,
        **({"roofline_cache_writes": {
            "kernels": "reshape_and_cache + hidden_to_cache + copy_blocks (prefill part of config 3)",
            "bound": "hbm", "bytes_per_step": st.prefill_write_bytes(), "ms_per_step": round(pf_ms, 4),
            "achieved": round(st.prefill_write_bytes() / (pf_ms * 1e-3) / 1e9, 1), "peak": peaks["hbm_gbs"],
            "unit": "GB/s", "frac": round(st.prefill_write_bytes() / (pf_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
            "prefill_tokens": int(w.prefill.meta.num_prefill_tokens),
            "copied_blocks": 0 if w.copy_pairs is None else int(w.copy_pairs.shape[0])}} if pf_ms else {}),
        "device_status": status,
    }
    if absorbed is not None:
        line["absorbed_variant"] = absorbed
    if cpu_baseline is not None:
        line["cpu_baseline"] = cpu_baseline
    print(json.dumps(line))
    if tp > 1:
        torch.distributed.destroy_process_group()


def run_reference(args):
    """The reference path's semantics on the host cores (the oracle port: the reference
    itself needs vLLM 0.5.0.post1 and a GPU), on a bounded sample of the same workload."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    # all host cores, also under torchrun (which exports OMP_NUM_THREADS=1 to its ranks)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    from apt_serve_b200.workloads import CONFIG_SHAPES, draw_decode_batch, make_decode_workload
    cfg = args.config
    shape = CONFIG_SHAPES[cfg]
    seed = 1000 + cfg
    lens, hid = draw_decode_batch(cfg, seed, batch=args.batch, hidden_fraction=args.hidden_fraction)
    hd = shape.num_heads * shape.head_dim
    sample = cpu_sample_requests(lens, hid, args.cpu_flops, shape.hidden, hd)
    # only the sampled requests are materialised on the host (same distributions, same seed)
    s_lens = [lens[r] for r in sample]
    s_hid = [hid[r] for r in sample]
    w = make_decode_workload(shape, s_lens, s_hid, seed, "cpu")
    reqs = list(range(len(sample)))
    sec = run_cpu_port(w, reqs, args.steps, min(args.warmup, 1))
    value = len(sample) / sec
    desc = (f"{len(sample)} of {len(lens)} requests of config {cfg} keeping the hidden/K-V mix "
            f"({sum(s_lens)} cached tokens) per step; tokens/s = sampled requests / time")
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT,
            "n_gpus": args.gpus, "steps": args.steps, "warmup": min(args.warmup, 1),
            "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True,
            "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"config {cfg}: {shape.name} layer, bounded sample", "seed": seed},
            "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": torch.get_num_threads(),
                             "host_cpus": os.cpu_count(), "kind": "port", "sample": desc},
            "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
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
    args = ap.parse_args()
    if args.impl == "reference":
        # bounded: the host cores do ~2 TFLOP/s, so K steps of the sample stay near two minutes
        args.cpu_flops = min(args.cpu_flops, 2.4e14 / max(1, args.steps))
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
