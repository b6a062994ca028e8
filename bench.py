"""Benchmark of the sparse hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4|c1|c2|c3|c5] [--impl reference]

A "step" is one pass of the hot path over one batch of synthetic input.  The default workload is
configuration 4, the largest one that fits a GPU and the one specified at 1/2/4/8 GPUs: a 2-layer
GCN forward on a 2 M-node power-law graph.  With N > 1 the graph's rows are split over the ranks by
stored entries and every layer all-gathers its dense features over NCCL inside the timed step
(strong scaling: the problem is fixed, the ranks share it).

One JSON line is printed by rank 0:
  value      device-resident throughput (inputs already in HBM), GFLOP/s over all ranks
  e2e        the same step from pinned host inputs to a pinned host result, copies inside
  roofline   for the kernel with the largest share of the step: algorithmic bytes per launch /
             mean launch duration (CUDA events inside the timed region) against the measured HBM
             copy bandwidth; `gather_model` beside it counts every gathered operand row as traffic
  phases     mean ms per step of the sharded forward's parts (dense transforms, SpMM launches,
             all-gathers on the communication stream, main-stream waits for gathered chunks)
  parity_check  sampled output rows of both sparse products of the timed forward against the
             float64 CPU oracle (the run exits non-zero when it fails)
  configs    (one GPU only) the other four configurations, each with its own step time, roofline
             and CPU baseline
  cpu_baseline  the reference's own OpenMP kernels (oracle/_ref, "reference") or the C port
             ("port") on this machine's host cores, on a bounded sample of the same workload
`--impl reference` times that CPU path as the whole run and prints the same line shape.

The K timed steps are repeated as blocks until the timed region is at least a second long; the
reported step time is that of the median block.
"""
from __future__ import annotations

import argparse
import datetime
import hashlib
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The CPU arm uses every host core this process may run on.  Launchers that start one process
# per GPU export OMP_NUM_THREADS=1; the OpenMP runtime reads the variable when it is first
# loaded (with torch), so it is corrected here, before that import.
_HOST_CORES = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
if "reference" in sys.argv[1:]:
    os.environ["OMP_NUM_THREADS"] = str(_HOST_CORES)
    os.environ.pop("OMP_PROC_BIND", None)

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "SpMM/SDDMM GFLOP/s"
UNIT = "GFLOP/s"
FALLBACK_HBM_GBS = 6650.0
RTOL, ATOL = 1e-4, 1e-5


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def ncu_traffic(workload: str, kernel: str):
    """DRAM bytes (read + write) per launch of `kernel` on `workload` from the profiler capture
    recorded in profiles/ncu_traffic.json, or None when there is no capture or the kernel's
    source file has changed since it was taken."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            table = json.load(f)["captures"]
    except Exception:
        return None
    for e in table:
        if e.get("workload") == workload and e.get("kernel") == kernel:
            try:
                with open(os.path.join(ROOT, e["source"]), "rb") as f:
                    if hashlib.sha256(f.read()).hexdigest() != e["source_sha256"]:
                        return None
            except Exception:
                return None
            return e.get("dram_bytes_per_launch")
    return None


def host_threads() -> dict:
    from oracle import oracle as O
    return {"os_cpu_count": os.cpu_count(), "affinity": _HOST_CORES,
            "torch_threads": torch.get_num_threads(), "openmp_threads": O.num_threads()}


# ---- clocks sampler ------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.gpu)], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                    power.append(float(parts[3]))
                except ValueError:
                    continue
                for name, flag in zip(names, parts[5:9]):
                    if flag.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        # "under load": samples taken while the GPU drew clearly more than its idle power
        load = [s for s, p in zip(sm, power) if p > 350.0] or sm
        return {"sm_mhz": statistics.median(load) if load else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm), "samples_under_load": len(load) if load is not sm else 0}


# ---- workloads -----------------------------------------------------------------------------------
class Workload:
    """What the measuring loop needs from a configuration."""
    name = ""
    units = 1
    kernels = ()
    launches_per_step = 1
    flush = None
    h2d_bytes = 0
    d2h_bytes = 0

    def run_info(self):
        return {}

    def e2e_step(self):
        raise NotImplementedError

    def begin_block(self):
        pass

    def stage_times(self, evs):
        return {name: statistics.mean(e[j].elapsed_time(e[j + 1]) for e in evs)
                for j, name in enumerate(self.kernels)}

    def extras(self, stage_ms):
        return {}

    def release(self):
        """Drop every tensor the workload holds (the next configuration gets the memory)."""
        import gc
        self.__dict__.clear()
        gc.collect()
        torch.cuda.empty_cache()


class SparseAttention(Workload):
    """Config 2: SDDMM + row softmax + SpMM, (batch*heads) independent units sharing one mask."""
    name = "c2_sparse_attention_seq4096_h8_d64_b4_band128_rand1pct"

    def __init__(self, batch=4, heads=8, seq=4096, d=64, window=128, density=0.01, world=1):
        self.batch, self.heads, self.seq, self.d = batch, heads, seq, d
        self.window, self.density = window, density
        self.units_total = batch * heads
        self.units = self.units_total     # this rank's share once set up
        self.world = world

    def host_inputs(self, units=None, rank=0):
        from scorch_b200 import workloads as W
        self.mask = W.attention_mask(self.seq, self.window, self.density, seed=0)
        self.nnz = self.mask.nnz
        if units is None:
            return W.attention_qkv(self.batch, self.heads, self.seq, self.d, seed=1 + rank)
        return W.attention_qkv(1, units, self.seq, self.d, seed=1 + rank)

    def setup(self, rank: int):
        from scorch_b200 import kernels as K, pipelines as P, sharded as S
        self.K = K
        Q, Km, V = self.host_inputs(rank=0)
        # the (batch, head) units are independent: each rank takes a contiguous share of them
        u0, u1 = S.unit_range(self.units_total, rank, self.world)
        self.units = u1 - u0
        Q, Km, V = (t[u0:u1].contiguous() for t in (Q, Km, V))
        self.host = [t.pin_memory() for t in (Q, Km, V)]
        self.host_out = torch.empty((self.units, self.seq, self.d), dtype=torch.float32).pin_memory()
        self.pos, self.crd, self.mval = (t.cuda() for t in (self.mask.pos, self.mask.crd, self.mask.val))
        self.Q, self.Km, self.V = (t.cuda() for t in self.host)
        self.plan = K.CsrPlan(self.pos, self.nnz)
        no_blocks = bool(os.environ.get("SCORCH_B200_NO_BLOCKS"))
        # the one-call attention path (what pipelines.sparse_attention picks for this mask); the
        # three-operator path is timed instead with SCORCH_B200_NO_FUSED=1
        self.attn_plan = (None if no_blocks or os.environ.get("SCORCH_B200_NO_FUSED")
                          else P.attention_plan(self.pos, self.crd, self.d, self.d))
        self.block_plan = None if no_blocks or self.attn_plan else P.attention_block_plan(self.pos, self.crd)
        self.band = isinstance(self.attn_plan, K.AttnBandPlan)
        if self.attn_plan:
            self.kernels = ("attn_scattered_kernel", "attn_band_kernel" if self.band else "attn_block_kernel")
        else:
            self.kernels = ("sddmm_kernel", "csr_row_softmax_kernel", "spmm_rows_kernel")
        self.scores = (None if self.attn_plan else
                       torch.empty((self.units, self.nnz), dtype=torch.float32, device="cuda"))
        self.out = torch.empty((self.units, self.seq, self.d), dtype=torch.float32, device="cuda")
        self.host_api = P.HostSparseAttention(self.pos, self.crd, self.mval, self.units, self.seq, self.d)

    @property
    def flops_total(self):  # SDDMM + SpMM, 2*nnz*d each (the reference tools' convention)
        return 2 * (2.0 * self.nnz * self.d) * self.units_total

    def config(self):
        return {"workload": self.name, "units": self.units_total, "seq": self.seq, "head_dim": self.d,
                "mask_nnz": self.nnz,
                "parallelism": f"(batch, head) units split over {self.world} GPU(s), no communication",
                "l2": "inputs larger than L2"}

    def run_info(self):
        bp = self.attn_plan or self.block_plan
        if self.band:
            return {"units_this_rank": self.units,
                    "path": "one attention call: scattered entries by the gather kernel, 128-row tiles x "
                            "384-column windows on tcgen05 (S, P and O in tensor memory; scores not stored)",
                    "entries_inside_windows": bp.inside, "entries_outside_windows": bp.rem_nnz}
        return {"units_this_rank": self.units,
                "path": ("one attention call (scattered entries and blocks share a running softmax; scores not stored)"
                         if self.attn_plan else "sddmm, row softmax, spmm"),
                "blocks_16x16": bp.blocks if bp else 0,
                "entries_outside_blocks": bp.rem_nnz if bp else self.nnz}

    def alg_bytes(self):
        """Algorithmic bytes per launch (each array read once / written once)."""
        nnz, s, d, u = self.nnz, self.seq, self.d, self.units
        idx = (s + 1) * 4 + nnz * 4
        if self.band:
            rem = self.attn_plan.rem_nnz
            rem_idx = (s + 1) * 4 + 2 * rem * 4
            return {
                "attn_scattered_kernel": rem_idx + rem * 4 + u * (4 * s * d * 4 + s * 8),
                # tiles: 12 mask words and the first entry per row, mask values of the window entries,
                # Q, K, V, unnormalised O and (maximum, sum) in, O out
                "attn_band_kernel": s * 13 * 4 + (nnz - rem) * 4 + u * (5 * s * d * 4 + s * 8),
            }
        if self.attn_plan:
            rem, blocks = self.attn_plan.rem_nnz, self.attn_plan.blocks
            rem_idx = (s + 1) * 4 + 2 * rem * 4          # rem_pos, rem_ent, crd of the listed entries
            return {
                # scattered entries: index lists, mask values, Q, K and V in; unnormalised O and
                # the rows' (maximum, sum) out
                "attn_scattered_kernel": rem_idx + rem * 4 + u * (4 * s * d * 4 + s * 8),
                # blocks: plan (column, first entry and mask per block row), mask values of the block
                # entries, Q, K, V, unnormalised O and (maximum, sum) in, O out
                "attn_block_kernel": blocks * (4 + 64 + 64) + (nnz - rem) * 4
                                     + u * (5 * s * d * 4 + s * 8),
            }
        return {
            "sddmm_kernel": idx + nnz * 4 + u * (2 * s * d * 4 + nnz * 4),
            "csr_row_softmax_kernel": (s + 1) * 4 + u * (2 * nnz * 4),
            "spmm_rows_kernel": idx + u * (nnz * 4 + 2 * s * d * 4),
        }

    def step(self, ev=None):
        K, Q, Km, V = self.K, self.Q, self.Km, self.V
        if ev is not None:
            ev[0].record()
        if self.attn_plan:
            # the attention call, kernel by kernel so that each can be timed (stages 1 and 2 of
            # kernels.sparse_attention_csr; together they are the default stages=3 call)
            for j, stage in enumerate((1, 2)):
                K.sparse_attention_csr(self.pos, self.crd, self.mval, Q, Km, V, attn_plan=self.attn_plan,
                                       out=self.out, stages=stage)
                if ev is not None:
                    ev[j + 1].record()
            return
        # same calls as pipelines.sparse_attention, with preallocated outputs
        s = K.sddmm_csr(self.pos, self.crd, self.mval, Q, Km, out=self.scores, block_plan=self.block_plan)
        if ev is not None:
            ev[1].record()
        K.csr_row_softmax(self.pos, s, out=s)
        if ev is not None:
            ev[2].record()
        K.spmm_csr(self.pos, self.crd, s, V, plan=self.plan, out=self.out, block_plan=self.block_plan)
        if ev is not None:
            ev[3].record()

    @property
    def launches_per_step(self):
        # with a block plan the SDDMM and SpMM stages of the three-operator path are two launches
        # each (tensor-core kernel over the dense blocks + gather kernel over the other entries)
        return 2 if self.attn_plan else (5 if self.block_plan else 3)

    def e2e_step(self):
        # the public host-tensor call: pinned Q, K, V in, pinned O out, copies inside
        self.host_api(*self.host, out_host=self.host_out)

    @property
    def h2d_bytes(self):
        return sum(t.numel() * 4 for t in self.host)

    @property
    def d2h_bytes(self):
        return self.host_out.numel() * 4

    def traffic_key(self):
        return self.name + ((":one_call_band" if self.band else ":one_call") if self.attn_plan else ":three_operators")

    # -- CPU reference on a bounded sample ---------------------------------------------------------
    def cpu_sample(self, units: int, repeats: int):
        """`units` heads through the reference's kernels: SDDMM (COO prebuilt, its fastest route),
        row softmax, SpMM.  Returns (GFLOP/s, kind, seconds, description)."""
        from oracle import oracle as O, ref_loader
        ref = ref_loader.load()
        pos, crd, mval = self.mask.pos, self.mask.crd, self.mask.val
        rows = torch.repeat_interleave(torch.arange(self.seq, dtype=torch.int32),
                                       (pos[1:] - pos[:-1]).long())
        Q, Km, V = (t[:units] for t in self.host)
        s, d, nnz = self.seq, self.d, self.nnz

        def one(u):
            if ref is not None:
                r = ref.sddmm_coo_float_prebuilt([s, s], [s, s], [[rows], [crd]], mval, [s, d], [[], []],
                                                 Q[u].reshape(-1), [s, d], [[], []], Km[u].reshape(-1))
                p = torch.from_numpy(O.csr_row_softmax(pos.numpy(), r.storage.value.numpy()))
                ref.spmm_csr_float_v2([s, d], [s, s], [[], [pos, crd]], p, [s, d], [[], []],
                                      V[u].reshape(-1), 256)
            else:
                v = O.sddmm_coo(rows.numpy(), crd.numpy(), mval.numpy(), Q[u].numpy(), Km[u].numpy())
                p = O.csr_row_softmax(pos.numpy(), v)
                O.spmm_csr_v2(pos.numpy(), crd.numpy(), p, V[u].numpy())

        one(0)  # warm-up
        t0 = time.perf_counter()
        for _ in range(repeats):
            for u in range(units):
                one(u)
        dt = (time.perf_counter() - t0) / repeats
        flops = 2 * (2.0 * nnz * d) * units
        kind = "reference" if ref is not None else "port"
        return flops / dt / 1e9, kind, dt, (f"{units} of {self.units_total} heads per step: sddmm_coo_float_prebuilt + "
                                            f"row softmax + spmm_csr_float_v2 ({kind})")


class SpmmWorkload(Workload):
    """Configs 1 and 3: one CSR x dense product."""

    def __init__(self, which: str, world: int = 1):
        self.which = which
        self.world = world
        self.name = {"c1": "c1_spmm_4096x4096_1pct_k64", "c3": "c3_sae_decode_8192x32768_top32_k4096"}[which]

    def setup(self, rank: int):
        from scorch_b200 import kernels as K, workloads as W
        self.K = K
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        if self.which == "c1":
            A = W.csr_uniform(4096, 4096, 0.01, seed=0)
            B = W.dense_normal(4096, 64, seed=1)
        else:
            A = W.sae_activations(8192, 32768, 32, seed=0, device=dev).to("cpu")
            B = W.sae_decoder(32768, 4096, seed=1, device=dev).cpu()
        self.A = A
        self.m_total, self.nnz_total = A.shape[0], A.nnz
        self.n, self.k = A.shape[1], B.shape[1]
        self.m, self.nnz = self.m_total, self.nnz_total
        self.host = [A.val, B]
        if dev == "cpu":
            return
        if self.world > 1:
            # rows of A balanced by stored entries, the dense operand held by every rank
            from scorch_b200 import sharded as S
            blk, self.bounds = S.row_block(A.pos, A.crd, A.val, rank, self.world)
            A = W.Csr((blk.rows, self.n), blk.pos, blk.crd, blk.val)
            self.m, self.nnz = blk.rows, blk.nnz
        self.host = [A.val.pin_memory(), B.pin_memory()]
        self.pos, self.crd = A.pos.cuda(), A.crd.cuda()
        self.val, self.B = (t.cuda() for t in self.host)
        self.stage = [torch.empty_like(t, device="cuda") for t in self.host]
        self.plan = K.CsrPlan(self.pos, self.nnz)
        self.out = torch.empty((self.m, self.k), dtype=torch.float32, device="cuda")
        self.host_out = torch.empty((self.m, self.k), dtype=torch.float32).pin_memory()
        # small problems stay in L2 between iterations: flush it with a 256 MiB write
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if self.which == "c1" else None

    @property
    def flops_total(self):
        return 2.0 * self.nnz_total * self.k

    def config(self):
        return {"workload": self.name, "m": self.m_total, "n": self.n, "k": self.k, "nnz": self.nnz_total,
                "parallelism": f"rows split by stored entries over {self.world} GPU(s), dense operand replicated",
                "l2": "L2 flushed by a 256 MiB write between iterations" if self.which == "c1"
                else "inputs larger than L2"}

    def run_info(self):
        return {"rows_this_rank": self.m, "nnz_this_rank": self.nnz}

    def alg_bytes(self):
        return {"spmm_rows_kernel": (self.m + 1) * 4 + self.nnz * 8 + self.n * self.k * 4 + self.m * self.k * 4}

    kernels = ("spmm_rows_kernel",)

    def step(self, ev=None):
        if self.flush is not None:
            self.flush.zero_()
        if ev is not None:
            ev[0].record()
        self.K.spmm_csr(self.pos, self.crd, self.val, self.B, plan=self.plan, out=self.out)
        if ev is not None:
            ev[1].record()

    def extras(self, stage_ms):
        ms = stage_ms["spmm_rows_kernel"]
        gm_bytes = self.nnz * (8 + self.k * 4) + self.m * self.k * 4
        out = {"gather_model": {"bytes": gm_bytes, "GBps": gm_bytes / (ms * 1e-3) / 1e9,
                                "what": "every stored entry counted as one operand-row read"}}
        if self.which == "c3":
            out["l2_gather"] = self.l2_gather_bound(ms)
        return out

    def l2_gather_bound(self, ms_default):
        """What bounds the wide product once DRAM traffic is the compulsory one: the rate at which
        the L2 hands 1 KB operand-row slices to the SMs.  Measured here with the library's probe
        kernel (random 1 KB rows of an L2-resident 32 MB panel, nothing else on the critical path)
        and compared with the product's own L2 -> SM volume (nnz * k * 4 bytes) per second, for the
        gather kernel and for the bulk-copy (cp.async.bulk through shared memory) kernel."""
        from scorch_b200 import _lib
        L = _lib.lib()
        st = torch.cuda.current_stream().cuda_stream

        def timed(fn, reps=5):
            fn()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            b.synchronize()
            return a.elapsed_time(b) / reps

        rows, warps, gathers = 32768, 148 * 64, 512
        panel = self.B[:, :256].contiguous()[:rows]
        sink = torch.zeros(warps, device="cuda", dtype=torch.float32)
        probe_ms = timed(lambda: _lib.check(L.sb_probe_l2_gather(panel.data_ptr(), panel.shape[0], gathers,
                                                                 warps, sink.data_ptr(), st)))
        peak = warps * gathers * 1024 / (probe_ms * 1e-3) / 1e9
        volume = self.nnz * self.k * 4
        per_kernel = {}
        before = L.sb_spmm_wide_select(-1)
        try:
            for name, mode in (("gather kernel (ld.global.nc.v8 through L1)", 0),
                               ("bulk-copy kernel (cp.async.bulk through shared memory)", 1)):
                L.sb_spmm_wide_select(mode)
                t = timed(lambda: self.K.spmm_csr(self.pos, self.crd, self.val, self.B, plan=self.plan,
                                                  out=self.out), reps=10)
                per_kernel[name] = {"ms": t, "l2_to_sm_GBps": volume / (t * 1e-3) / 1e9,
                                    "frac_of_probe": volume / (t * 1e-3) / 1e9 / peak}
        finally:
            L.sb_spmm_wide_select(before)
        return {"probe_GBps": peak, "probe": f"{warps} warps x {gathers} random 1 KB rows of a "
                f"{panel.shape[0]} x 256 fp32 panel (L2 resident)", "l2_to_sm_bytes_per_launch": volume,
                "kernels": per_kernel, "selected": "bulk-copy" if before == 1 else "gather",
                "wide_status": L.sb_spmm_wide_status()}

    def e2e_step(self):
        for dst, src in zip(self.stage, self.host):
            dst.copy_(src, non_blocking=True)
        self.K.spmm_csr(self.pos, self.crd, self.stage[0], self.stage[1], plan=self.plan, out=self.out)
        self.host_out.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    @property
    def h2d_bytes(self):
        return sum(t.numel() * 4 for t in self.host)

    @property
    def d2h_bytes(self):
        return self.m * self.k * 4

    def traffic_key(self):
        return self.name

    def cpu_sample(self, units: int, repeats: int):
        from oracle import oracle as O, ref_loader
        ref = ref_loader.load()
        A, B = self.A, self.host[1]

        def one():
            if ref is not None:
                ref.spmm_csr_float_v2([self.m_total, self.k], [self.m_total, self.n], [[], [A.pos, A.crd]], A.val,
                                      [self.n, self.k], [[], []], B.reshape(-1), 256)
            else:
                O.spmm_csr_v2(A.pos.numpy(), A.crd.numpy(), A.val.numpy(), B.numpy())
        one()
        t0 = time.perf_counter()
        for _ in range(repeats):
            one()
        dt = (time.perf_counter() - t0) / repeats
        kind = "reference" if ref is not None else "port"
        return self.flops_total / dt / 1e9, kind, dt, f"the whole product, spmm_csr_float_v2 ({kind})"


class SpgemmSpmv(Workload):
    """Config 5: SpMV sweep and SpGEMM C = A A on a 2M power-law matrix; symbolic and numeric
    phases timed separately.  Metric here: products (2 flops each) + SpMV flops per second."""
    name = "c5_spmspm_spmv_2M_powerlaw"
    SPMV_SWEEP = 10  # back-to-back SpMV calls per step: keeps the GPU busy between launches

    def __init__(self, n=2_000_000, world=1):
        self.n, self.world = n, world

    def setup(self, rank: int):
        from scorch_b200 import kernels as K, sharded as S, workloads as W
        self.K, self.S = K, S
        A = W.powerlaw_square(self.n, seed=0, device="cuda")
        self.A = A
        self.nnz = A.nnz
        self.x = W.randn_on((self.n,), seed=1, device="cuda")
        lens = (A.pos[1:] - A.pos[:-1]).long()
        self.products = int(lens[A.crd.long()].sum().item())
        # SpMV: rows balanced by stored entries; SpGEMM: rows of A balanced by products; the other
        # operand (x / the whole A) is held by every rank
        self.mv, _ = S.row_block(A.pos, A.crd, A.val, rank, self.world)
        self.mm, _ = S.row_block(A.pos, A.crd, A.val, rank, self.world,
                                 bounds=S.product_bounds(A.pos, A.crd, A.pos, self.world))
        self.timings = []

    @property
    def flops_total(self):
        return 2.0 * self.products + 2.0 * self.nnz * self.SPMV_SWEEP

    def config(self):
        return {"workload": self.name, "n": self.n, "nnz": self.nnz, "products": self.products,
                "spmv_calls_per_step": self.SPMV_SWEEP,
                "parallelism": f"SpMV rows split by stored entries, SpGEMM rows by products, over "
                               f"{self.world} GPU(s); x and the right operand replicated",
                "l2": "inputs larger than L2"}

    def run_info(self):
        return {"nnz_C_this_rank": getattr(self, "nnzc", None), "spmv_rows_this_rank": self.mv.rows,
                "spgemm_rows_this_rank": self.mm.rows}

    def alg_bytes(self):
        n, nnz = self.n, self.nnz
        nnzc = getattr(self, "nnzc", 0)
        mv, mm = self.mv, self.mm
        # per rank: its rows of the left operand, the replicated operand read once, its outputs
        return {"spmv": (mv.rows + 1) * 4 + mv.nnz * 8 + n * 4 + mv.rows * 4,
                "spgemm_symbolic": (mm.rows + 1) * 4 + mm.nnz * 4 + (n + 1) * 4 + nnz * 4 + (mm.rows + 1) * 4,
                "spgemm_numeric": (mm.rows + 1) * 4 + mm.nnz * 8 + (n + 1) * 4 + nnz * 8 + (mm.rows + 1) * 4
                                  + nnzc * 8}

    kernels = ("spmv", "spgemm_symbolic", "spgemm_numeric")
    launches_per_step = 12

    def begin_block(self):
        self.timings = []

    def step(self, ev=None):
        A, mv, mm = self.A, self.mv, self.mm
        if ev is not None:
            ev[0].record()
        for _ in range(self.SPMV_SWEEP):
            self.y = self.K.spmv_csr(mv.pos, mv.crd, mv.val, self.x)
        if ev is not None:
            ev[1].record()
        t = {}
        cpos, ccrd, cval = self.K.spgemm_csr(mm.pos, mm.crd, mm.val, A.pos, A.crd, A.val, self.n, timings=t)
        self.nnzc = int(ccrd.numel())
        if ev is not None:
            self.timings.append(t)
        del cpos, ccrd, cval

    def stage_times(self, evs):
        return {"spmv": statistics.mean(e[0].elapsed_time(e[1]) for e in evs) / self.SPMV_SWEEP,
                "spgemm_symbolic": statistics.mean(t["symbolic_ms"] for t in self.timings),
                "spgemm_numeric": statistics.mean(t["numeric_ms"] for t in self.timings)}

    def extras(self, stage_ms):
        return {"products_per_second": self.products / (stage_ms["spgemm_numeric"] * 1e-3)}

    def traffic_key(self):
        return self.name

    def cpu_sample(self, units: int, repeats: int):
        from oracle import oracle as O, ref_loader
        ref = ref_loader.load()
        # bounded sample: the first rows of A against the whole A
        rows = min(self.n, 50_000)
        pos = self.A.pos[: rows + 1].cpu()
        e = int(pos[-1])
        crd, val = self.A.crd[:e].cpu(), self.A.val[:e].cpu()
        Bp, Bc, Bv = self.A.pos.cpu(), self.A.crd.cpu(), self.A.val.cpu()
        lens = (Bp[1:] - Bp[:-1]).long()
        prods = int(lens[crd.long()].sum())
        t0 = time.perf_counter()
        if ref is not None:
            ref.prebuilt_spmspm_csr_f32([rows, self.n], [rows, self.n], [[], [pos, crd]], val,
                                        [self.n, self.n], [[], [Bp, Bc]], Bv)
        else:
            O.spgemm(pos.numpy(), crd.numpy(), val.numpy(), Bp.numpy(), Bc.numpy(), Bv.numpy(), self.n)
        dt = time.perf_counter() - t0
        kind = "reference" if ref is not None else "port"
        return 2.0 * prods / dt / 1e9, kind, dt, f"SpGEMM of the first {rows} rows of A with A ({kind})"


class GcnSharded(Workload):
    """Config 4: 2-layer GCN forward on a 2M-node power-law graph, rows sharded by nnz over the
    ranks; per layer the dense features are all-gathered (NCCL) in row chunks, each overlapped
    with the SpMM over the chunks that have arrived.  Strong scaling: the graph is fixed, the
    ranks split it."""
    K1, K2 = 256, 64
    CPU_SAMPLE_ROWS = 100_000

    def __init__(self, n=2_000_000, world=1):
        self.n, self.world = n, world
        self.name = ("c4_gcn_2M_powerlaw_k256_k64" if n == 2_000_000
                     else f"c4_gcn_{n}_nodes_powerlaw_k256_k64")

    # -- inputs ------------------------------------------------------------------------------------
    def graph(self):
        from scorch_b200 import workloads as W
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        g = W.gcn_graph(self.n, seed=0, device=dev)
        self.nnz_global = g.nnz
        self.max_row = int((g.pos[1:] - g.pos[:-1]).max().item())
        return g

    def weights(self, dev):
        from scorch_b200 import workloads as W
        return W.glorot(self.K1, self.K1, seed=0, device=dev), W.glorot(self.K1, self.K2, seed=1, device=dev)

    def take_cpu_sample_rows(self, g):
        ns = min(self.CPU_SAMPLE_ROWS, self.n)
        e = int(g.pos[ns])
        self.sample = (g.pos[:ns + 1].cpu(), g.crd[:e].cpu(), g.val[:e].cpu())

    def setup(self, rank: int):
        from scorch_b200 import sharded as S
        self.S = S
        self.rank = rank
        g = self.graph()
        self.shard = S.ShardedCsr.from_global(g.pos, g.crd, g.val, rank, self.world)
        r0, r1 = self.shard.bounds[rank], self.shard.bounds[rank + 1]
        if rank == 0 and self.world == 1:
            self.take_cpu_sample_rows(g)
        from scorch_b200 import pipelines as P
        self.W1, self.W2 = self.weights("cuda")
        # the host-tensor front end of the forward (what `e2e` times): its own split of the matrix
        self.host_api = P.HostGcnForward(g.pos, g.crd, g.val, self.W1, self.W2, rank, self.world)
        del g
        torch.cuda.empty_cache()
        gen = torch.Generator(device="cuda").manual_seed(1)
        X = torch.randn((self.n, self.K1), generator=gen, device="cuda", dtype=torch.float32)
        self.X = X[r0:r1].contiguous()
        del X
        torch.cuda.empty_cache()
        self.host_x = self.X.cpu().pin_memory()
        self.host_out = torch.empty((self.X.shape[0], self.K2), dtype=torch.float32).pin_memory()
        self.timeline = None

    @property
    def flops_total(self):  # the two sparse products (2*nnz*k) of the whole graph
        return 2.0 * self.nnz_global * (self.K1 + self.K2)

    def config(self):
        return {"workload": self.name, "nodes": self.n, "nnz": self.nnz_global, "max_row_nnz": self.max_row,
                "layers": "H = relu(A (X W1)), out = A (H W2); X 256 wide, W1 256x256, W2 256x64",
                "parallelism": f"rows sharded by stored entries over {self.world} GPU(s), "
                               "all-gather of the dense features per layer",
                "flops_counted": "2*nnz*(256+64), the two sparse products; the dense X*W products run "
                                 "inside the timed step but are not counted",
                "l2": "inputs larger than L2"}

    def run_info(self):
        sp = self.shard.splits
        segs = [b.plan.segments if b.plan is not None else None for b in sp[0].blocks]
        return {"rows_this_rank": self.shard.rows, "nnz_this_rank": self.shard.nnz,
                "row_chunk_offsets_layer1": sp[0].offsets, "row_chunk_offsets_layer2": sp[-1].offsets,
                "heavy_segments_per_chunk_layer1": segs}

    def alg_bytes(self):
        rows, nnz, n = self.shard.rows, self.shard.nnz, self.n
        per = lambda k: (rows + 1) * 4 + nnz * 8 + n * k * 4 + rows * k * 4
        return {"spmm_layer1_k256": per(self.K1), "spmm_layer2_k64": per(self.K2)}

    kernels = ("spmm_layer1_k256", "spmm_layer2_k64")

    @property
    def launches_per_step(self):
        # per layer one SpMM launch per row chunk (rows and heavy-row segments share the launch)
        return self.shard.splits[0].chunks + self.shard.splits[-1].chunks

    def begin_block(self):
        self.timeline = self.S.Timeline()

    def step(self, ev=None):
        self.out = self.S.gcn_forward_sharded(self.shard, self.X, self.W1, self.W2,
                                              timeline=self.timeline if ev is not None else None)

    def stage_times(self, evs):
        self.phases = self.timeline.summary()
        return {"spmm_layer1_k256": self.phases.get("spmm_layer1", 0.0),
                "spmm_layer2_k64": self.phases.get("spmm_layer2", 0.0)}

    def extras(self, stage_ms):
        nnz, rows = self.shard.nnz, self.shard.rows
        gm = {}
        for name, k in (("spmm_layer1_k256", self.K1), ("spmm_layer2_k64", self.K2)):
            b = nnz * (8 + 4 * k) + rows * k * 4
            gm[name] = {"bytes": b, "GBps": b / (stage_ms[name] * 1e-3) / 1e9 if stage_ms[name] else None}
        return {"gather_model": {"what": "every stored entry counted as one operand-row read "
                                         "(no reuse in cache); diagnostic, not the roofline numerator",
                                 **gm},
                "phases": {"ms_per_step": self.phases,
                           "what": "spmm_*, dense_transform and wait_for_gather are spans on the main "
                                   "stream (wait_for_gather = communication the pipeline did not hide); "
                                   "all_gather spans run on the communication stream"}}

    def e2e_step(self):
        # the public host-tensor call: pinned features in, pinned result rows out, copies inside
        self.host_api(self.host_x, self.host_out)

    @property
    def h2d_bytes(self):
        return self.host_x.numel() * 4

    @property
    def d2h_bytes(self):
        return self.host_out.numel() * 4

    def traffic_key(self):
        return self.name

    # -- parity of the timed forward ---------------------------------------------------------------
    def parity_check(self, reduce_max, reduce_sum, rows_total: int = 200):
        """Sampled rows (evenly spaced + this rank's longest) of both sparse products of the
        forward that was just timed, against the float64 oracle fed with the dense operand the
        GPU produced (the X W products are library GEMMs, outside the sparse path)."""
        from oracle import oracle as O
        S, shard = self.S, self.shard
        out = S.gcn_forward_sharded(shard, self.X, self.W1, self.W2)
        H = shard.buffer("hidden", (shard.rows, self.K1), self.X.device)
        loc = shard.local
        lens = (loc.pos[1:] - loc.pos[:-1]).long()
        per_rank = max(2, rows_total // self.world)
        rows = torch.unique(torch.cat([
            torch.linspace(0, shard.rows - 1, per_rank - 1, device=lens.device).long(),
            lens.argmax().reshape(1)]))
        starts, cnt = loc.pos[rows].long(), lens[rows]
        spos = torch.zeros(rows.numel() + 1, dtype=torch.int64, device=lens.device)
        spos[1:] = torch.cumsum(cnt, 0)
        idx = torch.repeat_interleave(starts - spos[:-1], cnt) + torch.arange(int(spos[-1]), device=lens.device)
        cols, inv = torch.unique(loc.crd[idx].long(), return_inverse=True)
        sval = loc.val[idx]
        worst, bad, checked = 0.0, 0, 0
        for operand_local, result, relu in ((torch.matmul(self.X, self.W1), H, True),
                                            (torch.matmul(H, self.W2), out, False)):
            full = S.gather_rows(shard, operand_local)
            sub = full[cols].cpu().numpy()
            del full
            want = O.spmm_csr_acc64(spos.to(torch.int32).cpu().numpy(), inv.to(torch.int32).cpu().numpy(),
                                    sval.cpu().numpy(), sub, None, relu)
            ok, err, nbad = O.allclose_report(result[rows].cpu().numpy(), want, RTOL, ATOL)
            worst, bad, checked = max(worst, float(err)), bad + int(nbad), checked + rows.numel()
        worst, bad, checked = reduce_max(worst), int(reduce_sum(bad)), int(reduce_sum(checked))
        return {"rows": checked, "max_abs_err": worst, "elements_outside_tolerance": bad, "ok": bad == 0,
                "tolerance": f"rtol {RTOL} / atol {ATOL} against float64 accumulation, per sparse product",
                "what": "rows of relu(A (X W1)) and of A (H W2) on every rank, longest row included"}

    # -- CPU reference on a bounded sample ---------------------------------------------------------
    def cpu_prepare(self):
        """Host operands of the CPU sample, allocated once outside any timed call."""
        pos, crd, val = self.sample
        rows = pos.numel() - 1
        gen = torch.Generator().manual_seed(2)
        self.cpu_ops = {
            "Xs": torch.randn((rows, self.K1), generator=gen, dtype=torch.float32),
            "T1": torch.randn((self.n, self.K1), generator=gen, dtype=torch.float32),
            "T2": torch.randn((self.n, self.K2), generator=gen, dtype=torch.float32),
            "W": self.weights("cpu"),
        }

    def cpu_sample(self, units: int, repeats: int):
        """The sample rows' share of one forward on the host: their dense transforms (torch) and
        both sparse products (the reference's spmm_csr_float_v2) against full-height operands."""
        from oracle import oracle as O, ref_loader
        ref = ref_loader.load()
        if not hasattr(self, "cpu_ops"):
            self.cpu_prepare()
        pos, crd, val = self.sample
        rows, n, ops = pos.numel() - 1, self.n, self.cpu_ops
        W1, W2 = ops["W"]

        def spmm(B, k):
            if ref is not None:
                r = ref.spmm_csr_float_v2([rows, k], [rows, n], [[], [pos, crd]], val, [n, k], [[], []],
                                          B.reshape(-1), 256)
                return r.storage.value.view(rows, k)
            return torch.from_numpy(O.spmm_csr_v2(pos.numpy(), crd.numpy(), val.numpy(), B.numpy()))

        def one():
            torch.matmul(ops["Xs"], W1)
            h = torch.relu_(spmm(ops["T1"], self.K1))
            torch.matmul(h, W2)
            spmm(ops["T2"], self.K2)

        one()  # warm-up: thread start-up and first touch stay outside the timed calls
        t0 = time.perf_counter()
        for _ in range(repeats):
            one()
        dt = (time.perf_counter() - t0) / repeats
        kind = "reference" if ref is not None else "port"
        flops = 2.0 * crd.numel() * (self.K1 + self.K2)
        return flops / dt / 1e9, kind, dt, (
            f"the first {rows} rows' share of one forward ({crd.numel()} stored entries): X W1, "
            f"spmm_csr_float_v2 k=256 + relu, H W2, spmm_csr_float_v2 k=64 ({kind}); operands "
            f"are full height ({n} rows)")


def make_workload(name: str, world: int = 1, c4_nodes: int = 2_000_000):
    if name == "c4":
        return GcnSharded(n=c4_nodes, world=world)
    if name == "c2":
        return SparseAttention(world=world)
    if name in ("c1", "c3"):
        return SpmmWorkload(name, world=world)
    if name == "c5":
        return SpgemmSpmv(world=world)
    raise SystemExit(f"unknown workload {name}")


# ---- measuring loop ----------------------------------------------------------------------------------
def measure(wl, K: int, W: int, world: int, barrier, max_over_ranks, min_seconds: float, max_blocks: int):
    """W warm-up steps, then blocks of exactly K steps (two events around each block, per-kernel
    events inside) until the blocks add up to `min_seconds`; returns the median block."""
    for _ in range(W):
        wl.step()
    nk = len(wl.kernels)
    blocks, total = [], 0.0
    while True:
        wl.begin_block()
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(nk + 1)] for _ in range(K)]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for i in range(K):
            wl.step(evs[i])
        end.record()
        barrier()
        block_ms = max_over_ranks(start.elapsed_time(end))
        total += block_ms
        if wl.flush is not None:
            # the L2 flush write sits between the per-kernel events, outside them
            block_ms = max_over_ranks(sum(e[0].elapsed_time(e[-1]) for e in evs))
        blocks.append((block_ms / K, wl.stage_times(evs)))
        if total >= min_seconds * 1e3 or len(blocks) >= max_blocks:
            break
    order = sorted(range(len(blocks)), key=lambda i: blocks[i][0])
    step_ms, stage_ms = blocks[order[len(order) // 2]]
    return step_ms, stage_ms, len(blocks), [b[0] for b in blocks]


def measure_e2e(wl, K: int, world: int, barrier, max_over_ranks):
    try:
        for _ in range(2):
            wl.e2e_step()
    except NotImplementedError:
        return None
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(K):
        wl.e2e_step()
    b.record()
    barrier()
    ms = max_over_ranks(a.elapsed_time(b)) / K
    return {"value": wl.flops_total / (ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ms,
            "steps": K, "h2d_bytes_per_step": wl.h2d_bytes, "d2h_bytes_per_step": wl.d2h_bytes}


def roofline_of(wl, stage_ms):
    peak, peak_kind = measured_peaks()
    alg = wl.alg_bytes()
    dom = max((k for k in stage_ms if stage_ms[k]), key=lambda k: stage_ms[k])
    achieved = alg[dom] / (stage_ms[dom] * 1e-3) / 1e9
    return {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "peak_source": peak_kind,
            "unit": "GB/s", "frac": achieved / peak, "frac_of_8TBps": achieved / 8000.0,
            "algorithmic_bytes_per_launch": alg[dom], "launch_ms": stage_ms[dom],
            "traffic": ncu_traffic(wl.traffic_key(), dom),
            "per_kernel": {k: {"ms": stage_ms[k], "algorithmic_GBps": (alg[k] / (stage_ms[k] * 1e-3) / 1e9)
                               if stage_ms[k] else None} for k in stage_ms}}


def cpu_baseline_of(wl, units: int, repeats: int):
    v, kind, dt, sample = wl.cpu_sample(units, repeats)
    return {"value": v, "unit": UNIT, "cores": host_threads()["openmp_threads"], "kind": kind,
            "sample": sample, "seconds_per_sample": dt, "threads": host_threads()}


# ---- reference arm --------------------------------------------------------------------------------
def run_reference(args, rank: int, emit):
    """The reference's CPU kernels as the whole run: every step is the bounded sample of the
    workload that `cpu_sample` describes, on all host cores."""
    if rank != 0:
        return
    torch.set_num_threads(_HOST_CORES)
    wl = make_workload(args.workload, args.gpus, args.c4_nodes)
    sample_units = 1
    if args.workload == "c2":
        sample_units = 2
        wl.host = list(wl.host_inputs(units=sample_units))
    elif args.workload == "c4":
        g = wl.graph()
        wl.take_cpu_sample_rows(g)
        del g
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        wl.cpu_prepare()
    else:
        wl.setup(0)
    for _ in range(max(0, args.warmup - 1)):   # (every sample call warms up once itself)
        wl.cpu_sample(sample_units, 1)
    vals, dts = [], []
    for _ in range(args.steps):
        v, kind, dt, sample = wl.cpu_sample(sample_units, 1)
        vals.append(v)
        dts.append(dt)
    value = statistics.median(vals)
    threads = host_threads()
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": statistics.median(dts) * 1e3,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": wl.config(),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads["openmp_threads"], "kind": kind,
                             "sample": sample, "threads": threads},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


def _bind_to_gpu_numa_node(index: int) -> None:
    """Run this rank (and allocate its pinned buffers) on the CPUs that sit next to its GPU: with
    one process per GPU the host-to-device copies of the end-to-end arm otherwise cross sockets."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception:
        pass


# ---- main -------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c4")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-units", type=int, default=2, help="heads in the CPU-baseline sample of c2")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true",
                    help="skip the other four configurations in the one-GPU line")
    ap.add_argument("--min-seconds", type=float, default=1.0,
                    help="repeat the block of K timed steps until the timed region is this long")
    ap.add_argument("--c4-nodes", type=int, default=2_000_000,
                    help="graph size of workload c4 (smaller graphs are for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # Libraries print banners to stdout (NCCL's version line): keep stdout for the one JSON line.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(line: dict):
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())

    if args.impl == "reference":
        run_reference(args, rank, emit)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); "
                         "use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    _bind_to_gpu_numa_node(local_rank)
    import torch.distributed as dist
    if world > 1:
        # (a rank that dies leaves the others in a collective: give up after four minutes, not ten)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank),
                                timeout=datetime.timedelta(seconds=240))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce(x: float, op) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=op)
        return float(t.item())

    max_over_ranks = lambda x: reduce(x, dist.ReduceOp.MAX)
    sum_over_ranks = lambda x: reduce(x, dist.ReduceOp.SUM)

    wl = make_workload(args.workload, world, args.c4_nodes)
    wl.setup(rank)
    K, W_ = args.steps, args.warmup

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    step_ms, stage_ms, nblocks, block_ms = measure(wl, K, W_, world, barrier, max_over_ranks,
                                                   args.min_seconds, 50)
    value = wl.flops_total / (step_ms * 1e-3) / 1e9
    scaling = "strong"   # every workload is a fixed problem that the ranks share
    e2e = measure_e2e(wl, min(K, 10) if args.workload == "c4" else K, world, barrier, max_over_ranks)
    clocks = sampler.stop() if rank == 0 else None

    roofline = roofline_of(wl, stage_ms)
    extras = wl.extras(stage_ms)
    parity = None
    if hasattr(wl, "parity_check"):
        parity = wl.parity_check(max_over_ranks, sum_over_ranks)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline = cpu_baseline_of(wl, args.cpu_units, 3 if args.workload in ("c1", "c2") else 1)

    line = None
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W_,
                "ms_per_step": step_ms, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "config": wl.config(), "run": wl.run_info(),
                "timed_blocks": {"blocks_of_K_steps": nblocks, "ms_per_step_each": block_ms,
                                 "reported": "median block"},
                "e2e": e2e, "gpu_launches": nblocks * K * wl.launches_per_step, "roofline": roofline,
                **extras, "parity_check": parity, "cpu_baseline": cpu_baseline, "clocks": clocks}

    # the other four configurations, one GPU only: each with its own step time, roofline, CPU arm
    if rank == 0 and world == 1 and args.workload == "c4" and not args.no_configs:
        wl.release()
        del wl
        configs = {}
        for name in ("c1", "c2", "c3", "c5"):
            w2 = make_workload(name)
            w2.setup(0)
            k2 = K if name != "c5" else min(K, 3)
            ms, st, nb, _ = measure(w2, k2, 3, 1, barrier, max_over_ranks, 0.3, 20)
            entry = {"config": w2.config(), "run": w2.run_info(), "ms_per_step": ms, "steps": k2, "blocks": nb,
                     "value": w2.flops_total / (ms * 1e-3) / 1e9, "unit": UNIT,
                     "roofline": roofline_of(w2, st), **w2.extras(st),
                     "e2e": measure_e2e(w2, min(k2, 10), 1, barrier, max_over_ranks)}
            if not args.no_cpu_baseline:
                entry["cpu_baseline"] = cpu_baseline_of(w2, args.cpu_units, 3 if name in ("c1", "c2") else 1)
            configs[name] = entry
            w2.release()
            del w2
        line["configs"] = configs

    if rank == 0:
        emit(line)
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        raise SystemExit("parity check of the timed forward failed: " + json.dumps(parity))


if __name__ == "__main__":
    main()
