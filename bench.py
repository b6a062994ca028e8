"""Benchmark of the sparse hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c1|c3|c4|c5] [--impl reference]

A "step" is one pass of the hot path over one batch of synthetic input.  The default workload is
the sparse-attention configuration (SDDMM -> row softmax -> SpMM over 4 x 8 heads, seq 4096,
head_dim 64, band-128 + 1 % random mask); with N > 1 every rank processes its own batch of the
same size (independent heads: no data-path collective, weak scaling).

One JSON line is printed by rank 0:
  value      device-resident throughput (inputs already in HBM), GFLOP/s over all ranks
  e2e        the same step through the public host-tensor API: pinned host inputs -> device,
             kernels, result -> host, all inside the timed region
  roofline   for the kernel with the largest share of the step: algorithmic bytes per launch /
             mean launch duration (CUDA events inside the timed region) against the measured
             HBM copy bandwidth
  cpu_baseline  the reference's own OpenMP kernels (oracle/_ref, "reference") or the C port
             ("port") on this machine's host cores, on a bounded sample of the same workload
`--impl reference` times that CPU path as the whole run and prints the same line shape.
"""
from __future__ import annotations

import argparse
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

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "SpMM/SDDMM GFLOP/s"
UNIT = "GFLOP/s"
FALLBACK_HBM_GBS = 6650.0

# DRAM bytes (read + write) per launch of each kernel from ncu captures of this benchmark's
# default workload, summarised under profiles/.  None = not captured yet.
NCU_TRAFFIC_BYTES = {
    "three operators": {
        "sddmm_kernel": 273_008_640,             # SDDMM stage: block kernel + remainder kernel
        "csr_row_softmax_kernel": 251_335_936,
        "spmm_rows_kernel": 319_077_120,         # SpMM stage: block kernel + remainder kernel
    },
    "one attention call": {
        "sddmm_kernel": 75_042_304,              # scores of the entries outside the blocks
        "attn_block_kernel": 147_454_720,
        "spmm_rows_kernel": 95_983_360,          # P V of the entries outside the blocks
    },
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


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
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, flag in zip(names, parts[5:9]):
                    if flag.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---- workloads -----------------------------------------------------------------------------------
class SparseAttention:
    """Config 2: SDDMM + row softmax + SpMM, (batch*heads) independent units sharing one mask."""
    name = "c2_sparse_attention_seq4096_h8_d64_b4_band128_rand1pct"

    def __init__(self, batch=4, heads=8, seq=4096, d=64, window=128, density=0.01):
        self.batch, self.heads, self.seq, self.d = batch, heads, seq, d
        self.window, self.density = window, density
        self.units = batch * heads

    def setup(self, rank: int):
        from scorch_b200 import kernels as K, workloads as W
        self.K = K
        self.mask = W.attention_mask(self.seq, self.window, self.density, seed=0)
        Q, Km, V = W.attention_qkv(self.batch, self.heads, self.seq, self.d, seed=1 + rank)
        self.host = [t.pin_memory() for t in (Q, Km, V)]
        self.host_out = torch.empty((self.units, self.seq, self.d), dtype=torch.float32).pin_memory()
        self.pos, self.crd, self.mval = (t.cuda() for t in (self.mask.pos, self.mask.crd, self.mask.val))
        self.Q, self.Km, self.V = (t.cuda() for t in self.host)
        self.nnz = self.mask.nnz
        self.plan = K.CsrPlan(self.pos, self.nnz)
        from scorch_b200 import pipelines as P
        no_blocks = bool(os.environ.get("SCORCH_B200_NO_BLOCKS"))
        # the one-call attention path (what pipelines.sparse_attention picks for this mask); the
        # three-operator path is timed instead with SCORCH_B200_NO_FUSED=1
        self.attn_plan = (None if no_blocks or os.environ.get("SCORCH_B200_NO_FUSED")
                          else P.attention_plan(self.pos, self.crd, self.d, self.d))
        self.block_plan = None if no_blocks or self.attn_plan else P.attention_block_plan(self.pos, self.crd)
        if self.attn_plan:
            self.kernels = ("sddmm_kernel", "attn_block_kernel", "spmm_rows_kernel")
        self.scores = (None if self.attn_plan else
                       torch.empty((self.units, self.nnz), dtype=torch.float32, device="cuda"))
        self.out = torch.empty((self.units, self.seq, self.d), dtype=torch.float32, device="cuda")
        from scorch_b200 import pipelines as P
        self.host_api = P.HostSparseAttention(self.pos, self.crd, self.mval, self.units, self.seq, self.d)

    @property
    def flops_per_step(self):  # SDDMM + SpMM, 2*nnz*d each (the reference tools' convention)
        return 2 * (2.0 * self.nnz * self.d) * self.units

    def config(self):
        bp = self.attn_plan or self.block_plan
        scores = 0 if self.attn_plan else self.units * self.nnz * 4
        return {"workload": self.name, "units_per_gpu": self.units, "seq": self.seq, "head_dim": self.d,
                "mask_nnz": self.nnz,
                "path": ("one attention call (blocks on tensor cores with running softmax; scores not stored)"
                         if self.attn_plan else "sddmm, row softmax, spmm"),
                "blocks_16x16": bp.blocks if bp else 0,
                "entries_outside_blocks": bp.rem_nnz if bp else self.nnz,
                "l2": "inputs larger than L2 (Q,K,V,O,scores,mask = "
                f"{(4 * self.units * self.seq * self.d * 4 + scores + self.nnz * 8) >> 20} MiB)"}

    def alg_bytes(self):
        """Algorithmic bytes per launch (each array read once / written once)."""
        nnz, s, d, u = self.nnz, self.seq, self.d, self.units
        idx = (s + 1) * 4 + nnz * 4
        if self.attn_plan:
            rem, blocks = self.attn_plan.rem_nnz, self.attn_plan.blocks
            rem_idx = (s + 1) * 4 + 2 * rem * 4          # rem_pos, rem_ent, crd of the listed entries
            return {
                # scores of the remaining entries: index lists, mask values, Q and K in, scores out
                "sddmm_kernel": rem_idx + rem * 4 + u * (2 * s * d * 4 + rem * 4),
                # blocks: plan (column, first entry and mask per block row), mask values of the block
                # entries, Q, K, V in, O out, remaining scores in / probabilities out
                "attn_block_kernel": blocks * (4 + 64 + 64) + (nnz - rem) * 4
                                     + u * (4 * s * d * 4 + 2 * rem * 4),
                # P V of the remaining entries: index lists, probabilities and V in, O in and out
                "spmm_rows_kernel": rem_idx + u * (rem * 4 + 3 * s * d * 4),
            }
        return {
            "sddmm_kernel": idx + nnz * 4 + u * (2 * s * d * 4 + nnz * 4),
            "csr_row_softmax_kernel": (s + 1) * 4 + u * (2 * nnz * 4),
            "spmm_rows_kernel": idx + u * (nnz * 4 + 2 * s * d * 4),
        }

    def _run(self, Q, Km, V, ev=None):
        K = self.K
        if ev is not None:
            ev[0].record()
        if self.attn_plan:
            # the attention call, kernel by kernel so that each can be timed (stages 1, 2, 4 of
            # kernels.sparse_attention_csr; together they are the default stages=7 call)
            for j, stage in enumerate((1, 2, 4)):
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

    # stage names; with a block plan the SDDMM and SpMM stages are two launches each
    # (tensor-core kernel over the dense blocks + gather kernel over the remaining entries)
    kernels = ("sddmm_kernel", "csr_row_softmax_kernel", "spmm_rows_kernel")

    @property
    def launches_per_step(self):
        return 5 if self.block_plan else 3   # (the attention call: 3 kernels)

    def step(self, ev=None):
        self._run(self.Q, self.Km, self.V, ev)

    def e2e_step(self):
        # the public host-tensor call: pinned Q, K, V in, pinned O out, copies inside
        self.host_api(*self.host, out_host=self.host_out)

    @property
    def h2d_bytes(self):
        return sum(t.numel() * 4 for t in self.host)

    @property
    def d2h_bytes(self):
        return self.host_out.numel() * 4

    # -- CPU reference on a bounded sample ---------------------------------------------------------
    def cpu_sample(self, units: int, repeats: int):
        """`units` heads through the reference's kernels: SDDMM (COO prebuilt, its fastest route),
        row softmax, SpMM.  Returns (GFLOP/s, description)."""
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
        return flops / dt / 1e9, kind, dt, (f"{units} of {self.units} heads per step: sddmm_coo_float_prebuilt + "
                                            f"row softmax + spmm_csr_float_v2 ({kind})")


class SpmmWorkload:
    """Configs 1 and 3: one CSR x dense product."""

    def __init__(self, which: str):
        self.which = which
        self.name = {"c1": "c1_spmm_4096x4096_1pct_k64", "c3": "c3_sae_decode_8192x32768_top32_k4096"}[which]
        self.units = 1

    def setup(self, rank: int):
        from scorch_b200 import kernels as K, workloads as W
        self.K = K
        if self.which == "c1":
            A = W.csr_uniform(4096, 4096, 0.01, seed=0)
            B = W.dense_normal(4096, 64, seed=1)
        else:
            A = W.sae_activations(8192, 32768, 32, seed=0, device="cuda").to("cpu")
            B = W.sae_decoder(32768, 4096, seed=1, device="cuda").cpu()
        self.A = A
        self.m, self.n, self.k, self.nnz = A.shape[0], A.shape[1], B.shape[1], A.nnz
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
    def flops_per_step(self):
        return 2.0 * self.nnz * self.k

    def config(self):
        return {"workload": self.name, "m": self.m, "n": self.n, "k": self.k, "nnz": self.nnz,
                "l2": "L2 flushed by a 256 MiB write between iterations" if self.flush is not None
                else "inputs larger than L2"}

    def alg_bytes(self):
        return {"spmm_rows_kernel": (self.m + 1) * 4 + self.nnz * 8 + self.n * self.k * 4 + self.m * self.k * 4}

    kernels = ("spmm_rows_kernel",)
    launches_per_step = 1

    def step(self, ev=None):
        if self.flush is not None:
            self.flush.zero_()
        if ev is not None:
            ev[0].record()
        self.K.spmm_csr(self.pos, self.crd, self.val, self.B, plan=self.plan, out=self.out)
        if ev is not None:
            ev[1].record()

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
        return self.host_out.numel() * 4

    def cpu_sample(self, units: int, repeats: int):
        from oracle import oracle as O, ref_loader
        ref = ref_loader.load()
        A, B = self.A, self.host[1]

        def one():
            if ref is not None:
                ref.spmm_csr_float_v2([self.m, self.k], [self.m, self.n], [[], [A.pos, A.crd]], A.val,
                                      [self.n, self.k], [[], []], B.reshape(-1), 256)
            else:
                O.spmm_csr_v2(A.pos.numpy(), A.crd.numpy(), A.val.numpy(), B.numpy())
        one()
        t0 = time.perf_counter()
        for _ in range(repeats):
            one()
        dt = (time.perf_counter() - t0) / repeats
        kind = "reference" if ref is not None else "port"
        return self.flops_per_step / dt / 1e9, kind, dt, f"the whole product, spmm_csr_float_v2 ({kind})"


class SpgemmSpmv:
    """Config 5: SpMV sweep and SpGEMM C = A A on a 2M power-law matrix; symbolic and numeric
    phases timed separately.  Metric here: products (2 flops each) + SpMV flops per second."""
    name = "c5_spmspm_spmv_2M_powerlaw"

    def __init__(self, n=2_000_000):
        self.n = n
        self.units = 1

    def setup(self, rank: int):
        from scorch_b200 import kernels as K, workloads as W
        self.K = K
        A = W.powerlaw_square(self.n, seed=0, device="cuda")
        self.A = A
        self.nnz = A.nnz
        self.x = W.randn_on((self.n,), seed=1, device="cuda")
        self.plan = K.CsrPlan(A.pos, self.nnz)
        lens = (A.pos[1:] - A.pos[:-1]).long()
        self.products = int(lens[A.crd.long()].sum().item())
        self.timings = {}

    @property
    def flops_per_step(self):
        return 2.0 * self.products + 2.0 * self.nnz * self.SPMV_SWEEP

    def config(self):
        return {"workload": self.name, "n": self.n, "nnz": self.nnz, "products": self.products,
                "spmv_calls_per_step": self.SPMV_SWEEP,
                "l2": "inputs larger than L2"}

    def alg_bytes(self):
        n, nnz = self.n, self.nnz
        nnzc = getattr(self, "nnzc", 0)
        return {"spmv": (n + 1) * 4 + nnz * 8 + 2 * n * 4,
                "spgemm_symbolic": (n + 1) * 4 + nnz * 4 + (n + 1) * 4,
                "spgemm_numeric": (n + 1) * 4 + nnz * 8 + (n + 1) * 4 + nnzc * 8}

    kernels = ("spmv", "spgemm_symbolic", "spgemm_numeric")
    launches_per_step = 12

    SPMV_SWEEP = 10  # back-to-back SpMV calls per step: keeps the GPU busy between launches

    def step(self, ev=None):
        A = self.A
        if ev is not None:
            ev[0].record()
        for _ in range(self.SPMV_SWEEP):
            self.y = self.K.spmv_csr(A.pos, A.crd, A.val, self.x, plan=self.plan)
        if ev is not None:
            ev[1].record()
        t = {}
        cpos, ccrd, cval = self.K.spgemm_csr(A.pos, A.crd, A.val, A.pos, A.crd, A.val, self.n, timings=t)
        self.nnzc = int(ccrd.numel())
        self.timings = t
        del cpos, ccrd, cval

    def e2e_step(self):
        raise NotImplementedError

    h2d_bytes = 0
    d2h_bytes = 0

    def cpu_sample(self, units: int, repeats: int):
        from oracle import oracle as O, ref_loader
        ref = ref_loader.load()
        # bounded sample: the first 100k rows of A against the whole A
        rows = min(self.n, 100_000)
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


class GcnSharded:
    """Config 4: 2-layer GCN forward on a 2M-node power-law graph, rows sharded by nnz over the
    ranks; per layer the dense features are all-gathered (NCCL) panel by panel, overlapped with
    the SpMM of earlier panels.  Strong scaling: the graph is fixed, ranks split it."""
    name = "c4_gcn_2M_powerlaw_k256_k64"

    def __init__(self, n=2_000_000, world=1):
        self.n, self.world = n, world
        self.units = 1

    def setup(self, rank: int):
        from scorch_b200 import kernels as K, sharded as S, workloads as W
        self.S = S
        g = W.gcn_graph(self.n, seed=0, device="cuda")
        self.nnz_global = g.nnz
        self.shard = S.ShardedCsr.from_global(g.pos, g.crd, g.val, rank, self.world)
        self.max_row = int((g.pos[1:] - g.pos[:-1]).max().item())
        r0, r1 = self.shard.bounds[rank], self.shard.bounds[rank + 1]
        if rank == 0:
            ns = min(100_000, self.n)
            self.sample = (g.pos[:ns + 1].cpu(), g.crd[:int(g.pos[ns])].cpu(), g.val[:int(g.pos[ns])].cpu())
        del g
        torch.cuda.empty_cache()
        gen = torch.Generator(device="cuda").manual_seed(1)
        X = torch.randn((self.n, 256), generator=gen, device="cuda", dtype=torch.float32)
        self.X = X[r0:r1].contiguous()
        del X
        torch.cuda.empty_cache()
        self.W1, self.W2 = W.glorot(256, 256, seed=0, device="cuda"), W.glorot(256, 64, seed=1, device="cuda")
        self.panel = None if self.world == 1 else "32,32,64,... (layer 1), 32,32 (layer 2)"
        self.host_x = self.X.cpu().pin_memory()
        self.stage_x = torch.empty_like(self.X)
        self.host_out = torch.empty((self.X.shape[0], 64), dtype=torch.float32).pin_memory()
        self.spmm_ms = []
        self._ev = []

    @property
    def flops_per_step(self):  # the two sparse products (2*nnz*k); per-rank share is 1/world
        return 2.0 * self.nnz_global * (256 + 64) / self.world

    def config(self):
        return {"workload": self.name, "nodes": self.n, "nnz": self.nnz_global, "max_row_nnz": self.max_row,
                "rows_this_rank": self.shard.rows, "heavy_segments_this_rank": self.shard.plan.segments
                if self.shard.plan else None, "panel": self.panel or "full width",
                "parallelism": f"row-sharded x{self.world}, all-gather per layer",
                "flops_counted": "2*nnz*(256+64), the two sparse products; dense X*W GEMMs run inside "
                                 "the timed step but are not counted", "l2": "inputs larger than L2"}

    def alg_bytes(self):
        rows, nnz, n = self.shard.rows, self.shard.nnz, self.n
        per = lambda k: (rows + 1) * 4 + nnz * 8 + n * k * 4 + rows * k * 4
        return {"spmm_layer1_k256": per(256), "spmm_layer2_k64": per(64)}

    kernels = ("spmm_layer1_k256", "spmm_layer2_k64")

    @property
    def launches_per_step(self):
        # SpMM calls per forward (one per column panel; 2 with one rank, 4 with two, 7 beyond) x
        # kernels per call (rows kernel, + heavy-segment kernel and its fix-up when the block has heavy rows)
        calls = 2 if self.world == 1 else (4 + 1 if self.world == 2 else 5 + 2)
        per_call = 3 if (self.shard.plan is not None and self.shard.plan.segments) else 1
        return calls * per_call

    def _spmm_timed(self, shard, B, out, relu):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        self.S._default_spmm(shard, B, out, relu)
        b.record()
        self._ev.append((relu, a, b))

    def _forward(self, x, timed=False):
        return self.S.gcn_forward_sharded(self.shard, x, self.W1, self.W2,
                                          spmm_fn=self._spmm_timed if timed else None)

    def step(self, ev=None):
        if ev is not None:
            self._timed_steps = getattr(self, "_timed_steps", 0) + 1
        self.out = self._forward(self.X, timed=ev is not None)

    def stage_times(self):
        # a layer is several SpMM launches when it runs in column panels: sum them per step
        l1 = [a.elapsed_time(b) for relu, a, b in self._ev if relu]
        l2 = [a.elapsed_time(b) for relu, a, b in self._ev if not relu]
        steps = max(1, getattr(self, "_timed_steps", 0))
        return {"spmm_layer1_k256": sum(l1) / steps, "spmm_layer2_k64": sum(l2) / steps}

    def e2e_step(self):
        self.stage_x.copy_(self.host_x, non_blocking=True)
        out = self._forward(self.stage_x)
        self.host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    @property
    def h2d_bytes(self):
        return self.host_x.numel() * 4

    @property
    def d2h_bytes(self):
        return self.host_out.numel() * 4

    def cpu_sample(self, units: int, repeats: int):
        from oracle import oracle as O, ref_loader
        ref = ref_loader.load()
        pos, crd, val = self.sample
        rows, n, k = pos.numel() - 1, self.n, 256
        B = torch.randn((n, k), dtype=torch.float32)
        t0 = time.perf_counter()
        if ref is not None:
            ref.spmm_csr_float_v2([rows, k], [rows, n], [[], [pos, crd]], val, [n, k], [[], []], B.reshape(-1), 256)
        else:
            O.spmm_csr_v2(pos.numpy(), crd.numpy(), val.numpy(), B.numpy())
        dt = time.perf_counter() - t0
        kind = "reference" if ref is not None else "port"
        return 2.0 * crd.numel() * k / dt / 1e9, kind, dt, (f"layer-1 SpMM (k=256) of the first {rows} rows "
                                                           f"({crd.numel()} entries), spmm_csr_float_v2 ({kind})")


def make_workload(name: str, world: int = 1, c4_nodes: int = 2_000_000):
    if name == "c4":
        return GcnSharded(n=c4_nodes, world=world)
    if name == "c2":
        return SparseAttention()
    if name in ("c1", "c3"):
        return SpmmWorkload(name)
    if name == "c5":
        return SpgemmSpmv()
    raise SystemExit(f"unknown workload {name}")


# ---- reference arm --------------------------------------------------------------------------------
def run_reference(args, rank: int, emit):
    if rank != 0:
        return
    wl = make_workload(args.workload, 1, args.c4_nodes)
    if args.workload == "c2":
        # build host inputs only (no CUDA needed for this arm)
        from scorch_b200 import workloads as W
        wl.mask = W.attention_mask(wl.seq, wl.window, wl.density, seed=0)
        wl.nnz = wl.mask.nnz
        sample_units = 2
        Q, Km, V = W.attention_qkv(1, sample_units, wl.seq, wl.d, seed=1)
        wl.host = [Q, Km, V]
        cfg = {"workload": wl.name, "units_per_gpu": wl.units, "seq": wl.seq, "head_dim": wl.d,
               "mask_nnz": wl.nnz}
    else:
        wl.setup(0)
        sample_units = 1
        cfg = wl.config()
    for _ in range(max(1, args.warmup) - 1):
        wl.cpu_sample(sample_units, 1)
    vals, dts = [], []
    for _ in range(args.steps):
        v, kind, dt, sample = wl.cpu_sample(sample_units, 1)
        vals.append(v)
        dts.append(dt)
    from oracle import oracle as O
    value = statistics.median(vals)
    cores = max(torch.get_num_threads(), O.num_threads())
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": statistics.median(dts) * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
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
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-units", type=int, default=2, help="heads in the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    wl = make_workload(args.workload, world, args.c4_nodes)
    wl.setup(rank)
    K, W_ = args.steps, args.warmup

    for _ in range(W_):
        wl.step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    # device-resident arm: K steps between two events; per-kernel events inside the region
    nk = len(wl.kernels)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(nk + 1)] for _ in range(K)]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for i in range(K):
        wl.step(evs[i])
    end.record()
    barrier()
    total_ms = max_over_ranks(start.elapsed_time(end))
    flush_ms = 0.0
    if getattr(wl, "flush", None) is not None:
        # the L2 flush write sits between the per-kernel events, outside them: take it out of the step time
        flush_ms = total_ms - sum(e[0].elapsed_time(e[-1]) for e in evs)
    step_ms = (total_ms - flush_ms) / K
    stage_ms = {}
    if args.workload == "c4":
        stage_ms = wl.stage_times()
    elif args.workload == "c5":
        stage_ms = {"spmv": statistics.mean(e[0].elapsed_time(e[1]) for e in evs) / wl.SPMV_SWEEP,
                    "spgemm_symbolic": wl.timings.get("symbolic_ms"), "spgemm_numeric": wl.timings.get("numeric_ms")}
    else:
        for j, name in enumerate(wl.kernels):
            stage_ms[name] = statistics.mean(e[j].elapsed_time(e[j + 1]) for e in evs)
    value = wl.flops_per_step * world / (step_ms * 1e-3) / 1e9
    scaling = "strong" if args.workload == "c4" else "weak"

    # end-to-end arm through host tensors
    e2e = None
    try:
        for _ in range(2):
            wl.e2e_step()
        barrier()
        t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_start.record()
        for _ in range(K):
            wl.e2e_step()
        t_end.record()
        barrier()
        e2e_ms = max_over_ranks(t_start.elapsed_time(t_end)) / K
        e2e = {"value": wl.flops_per_step * world / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
               "ms_per_step": e2e_ms, "h2d_bytes_per_step": wl.h2d_bytes, "d2h_bytes_per_step": wl.d2h_bytes}
    except NotImplementedError:
        e2e = None
    clocks = sampler.stop() if rank == 0 else None

    peak, peak_kind = measured_peaks()
    alg = wl.alg_bytes()
    dom = max((k for k in stage_ms if stage_ms[k]), key=lambda k: stage_ms[k])
    achieved = alg[dom] / (stage_ms[dom] * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "peak_source": peak_kind,
                "unit": "GB/s", "frac": achieved / peak, "algorithmic_bytes_per_launch": alg[dom],
                "launch_ms": stage_ms[dom],
                "traffic": (NCU_TRAFFIC_BYTES["one attention call" if wl.attn_plan else "three operators"].get(dom)
                            if args.workload == "c2" else None),
                "per_kernel": {k: {"ms": stage_ms[k], "algorithmic_GBps": (alg[k] / (stage_ms[k] * 1e-3) / 1e9)
                                   if stage_ms[k] else None} for k in stage_ms}}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import oracle as O
        v, kind, dt, sample = wl.cpu_sample(args.cpu_units, 3 if args.workload == "c2" else 1)
        cpu_baseline = {"value": v, "unit": UNIT, "cores": max(torch.get_num_threads(), O.num_threads()),
                        "kind": kind, "sample": sample, "seconds_per_sample": dt}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W_,
                "ms_per_step": step_ms, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "config": wl.config(), "e2e": e2e,
                "gpu_launches": K * wl.launches_per_step, "roofline": roofline, "cpu_baseline": cpu_baseline,
                "clocks": clocks}
        emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
