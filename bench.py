"""Benchmark of the decode hot path: one Llama-3-8B-shaped decode layer step, batched variable-length.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (BASELINE.json configs[2]): hidden 4096, 32 q heads / 8 kv heads, head_dim 128, FFN 14336 with Q8_0
weights, FP16 attention weights, batch 32 with per-sequence contexts uniform in [512, 8192], RoPE theta 5e5.
One step = one pass of the layer over the batch (fused norm+QKV+RoPE+append+batched decode attention, then
output projection + residual, norm, Q8_0 SwiGLU FFN + residual): 32 tokens advance one layer.

`value`   tokens/s with inputs resident in HBM, the layer replayed as one CUDA graph on the decode stream.
`e2e`     the same metric through the C ABI with HOST buffers: per step the activations and the batch plan are
          copied from pinned host memory, the layer runs, the result is copied back; two steps in flight (the next
          step's upload and the previous step's download overlap the compute), the one-call-at-a-time figure beside it.
`roofline` the dominant kernel (batched decode attention): algorithmic bytes / CUDA-event duration vs the
          measured HBM copy bandwidth.
`cpu_baseline` the oracle (CPU restatement of the reference math) timed on this box's host cores on a bounded
          sample of the same batch.
`parity`  before any timing one eager step of the exact batch is compared with the oracle on four rows (shortest,
          longest and two more): layer output and the appended K/V rows. A miss ends the run with exit code 3.
With N > 1 (torchrun) ONE global batch of 32 x N sequences is dealt to the ranks, longest first onto the least
loaded rank with 32 sequences each (weak scaling, no collective on the path); the slowest rank sets the step time.
"""
from __future__ import annotations

import argparse
import ctypes as C
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
PKG_DIR = os.path.join(ROOT, "m40-llm_b200")

H, QH, KVH, HD, F = 4096, 32, 8, 128, 14336
B, LMIN, LMAX = 32, 512, 8192
EPS, THETA = 1e-5, 500000.0
N_WEIGHT_SETS = 2  # rotated between steps so no weight byte survives in L2 from one step to the next
# Traffic of the dominant kernel from the committed ncu capture (profiles/): DRAM bytes per algorithmic byte.
NCU_TRAFFIC_RATIO = 1.03
CPU_BASELINE_SECONDS = 12.0  # wall time spent in the oracle for the cpu_baseline leg
MIN_TIMED_SECONDS = 0.3      # a timed loop repeats its block of `steps` until it has run at least this long
ATOL, RTOL = 1e-3, 2e-3      # parity tolerance: |a - e| <= ATOL + RTOL * |e|


def load_package():
    """The package directory carries a hyphen, so it is loaded by path."""
    if "m40_llm_b200" in sys.modules:
        return sys.modules["m40_llm_b200"]
    spec = importlib.util.spec_from_file_location(
        "m40_llm_b200", os.path.join(PKG_DIR, "__init__.py"), submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["m40_llm_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def layer_weight_bytes():
    attn = (QH * HD * H + 2 * KVH * HD * H + H * QH * HD) * 2
    ffn = (2 * F * (H // 32) * 34) + H * (F // 32) * 34
    return attn + ffn


def attention_bytes(lens):
    # K and V once per kv head, q and out once (f32)
    return int(sum(2 * int(l) * KVH * HD * 2 for l in lens) + len(lens) * 2 * QH * HD * 4)


def step_bytes(lens):
    rows = len(lens)
    act = rows * H * 4 * 8  # x, xn, q, att, x1, x1n, out and the hid round trip are small next to weights
    return layer_weight_bytes() + attention_bytes(lens) + act


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")] + [time.perf_counter()])

    def wait_first_sample(self, timeout=5.0):
        t0 = time.perf_counter()
        while not self.rows and time.perf_counter() - t0 < timeout:
            time.sleep(0.01)

    def mark(self):
        return time.perf_counter()

    def stop(self, t_begin=None, t_end=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = self.rows
        if t_begin is not None:  # samples taken while the timed loop ran (one sample of slack either side)
            inside = [r for r in rows if t_begin - 0.03 <= r[-1] <= t_end + 0.03]
            rows = inside or rows[-3:]
        sm = [float(r[0]) for r in rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in rows if len(r) >= 7 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def make_inputs(O, world):
    """ONE global batch of B * world sequences (lengths, activations) and the layer weights, all from fixed seeds, so
    that every rank derives the same batch and the same weights (weights are replicated, sequences are dealt)."""
    rng = np.random.default_rng(0)
    lens = rng.integers(LMIN, LMAX + 1, size=B * world).astype(np.uint32)
    sets = []
    for _ in range(N_WEIGHT_SETS):
        w = {}
        for n, s in dict(wq=(QH * HD, H), wk=(KVH * HD, H), wv=(KVH * HD, H), wo=(H, QH * HD)).items():
            w[n] = (rng.standard_normal(s, dtype=np.float32) * 0.02).astype(np.float16)
        for n, s in dict(wg=(F, H), wu=(F, H), wd=(H, F)).items():
            w[n] = O.q80_quantize(rng.standard_normal(s, dtype=np.float32) * np.float32(0.02))
        w["attn_norm"] = np.ones(H, np.float32)
        w["ffn_norm"] = np.ones(H, np.float32)
        sets.append(w)
    x = np.random.default_rng(77).standard_normal((B * world, H), dtype=np.float32)
    return lens, sets, x


def kv_for_sequence(global_index, n):
    """Cache contents of one sequence of the global batch (seeded by its index, whichever rank it lands on)."""
    rng = np.random.default_rng(1000 + int(global_index))
    k = rng.standard_normal((n, KVH, HD), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((n, KVH, HD), dtype=np.float32).astype(np.float16)
    return k, v


def timed_blocks(launch_block, events, steps, pilot_ms):
    """Times `blocks` repetitions of a block of `steps` launches inside ONE event bracket, with `blocks` chosen from
    a pilot block so that the bracket lasts at least MIN_TIMED_SECONDS. Returns (ms per step, blocks)."""
    blocks = max(1, int(np.ceil(MIN_TIMED_SECONDS * 1e3 / max(pilot_ms, 1e-3))))
    events.start()
    for b in range(blocks):
        launch_block(b * steps)
    return events.stop_ms() / (blocks * steps), blocks


class Layer:
    """Issues one decode layer step through the C ABI (everything on the decode stream)."""

    def __init__(self, nat, kv, dw, rows):
        self.nat, self.kv, self.dw, self.rows = nat, kv, dw, rows
        self.dx = nat.buf(rows * H * 4)
        self.dq = nat.buf(rows * QH * HD * 4)
        self.datt = nat.buf(rows * QH * HD * 4)
        self.dx1 = nat.buf(rows * H * 4)
        self.dx1n = nat.buf(rows * H * 4)
        self.dhid = nat.buf(rows * F * 4)
        self.dout = nat.buf(rows * H * 4)
        self.dids = nat.buf(rows * 4)
        self.dpos = nat.buf(rows * 4)
        self.dlens = nat.buf(rows * 4)

    def enqueue(self, wset):
        L, ctx, d, r = self.nat.lib, self.nat.ctx, self.dw[wset], self.rows
        rc = L.m40llm_qkv_rope_append_attention_async(ctx, self.kv, self.dx.ptr, d["attn_norm"].ptr, 1, EPS, d["wq"].ptr,
                                                      d["wk"].ptr, d["wv"].ptr, None, None, None, self.dids.ptr,
                                                      self.dpos.ptr, self.dlens.ptr, r, H, QH, THETA, 1.0, 0, self.dq.ptr,
                                                      self.datt.ptr)
        assert rc == 0, rc
        rc = L.m40llm_attn_out_ffn_async(ctx, self.datt.ptr, d["wo"].ptr, self.dx.ptr, d["ffn_norm"].ptr, 1, EPS,
                                         d["wg"].ptr, d["wu"].ptr, d["wd"].ptr, 1, self.dx1.ptr, self.dhid.ptr,
                                         self.dout.ptr, r, H, QH * HD, F)
        assert rc == 0, rc

    def attention_only(self):
        L = self.nat.lib
        rc = L.m40llm_attention_last_token_f32_gqa_batched_async(self.nat.ctx, self.kv, self.dids.ptr, self.dlens.ptr,
                                                                 self.rows, self.dq.ptr, QH, self.datt.ptr)
        assert rc == 0, rc

    def capture(self, wset):
        L, ctx = self.nat.lib, self.nat.ctx
        assert L.m40llm_cuda_graph_begin_capture(ctx, 1) == 0
        self.enqueue(wset)
        g = C.c_void_p()
        assert L.m40llm_cuda_graph_end_capture(ctx, 1, C.byref(g)) == 0 and g.value
        return g


class Events:
    def __init__(self, nat):
        self.nat = nat
        self.e0, self.e1 = C.c_void_p(), C.c_void_p()
        assert nat.lib.m40llm_cuda_event_create(nat.ctx, C.byref(self.e0)) == 0
        assert nat.lib.m40llm_cuda_event_create(nat.ctx, C.byref(self.e1)) == 0

    def start(self):
        assert self.nat.lib.m40llm_cuda_event_record(self.nat.ctx, self.e0, 1) == 0

    def stop_ms(self):
        assert self.nat.lib.m40llm_cuda_event_record(self.nat.ctx, self.e1, 1) == 0
        ms = C.c_float()
        assert self.nat.lib.m40llm_cuda_event_elapsed_sync(self.nat.ctx, self.e0, self.e1, C.byref(ms)) == 0
        return float(ms.value)


def launches(nat):
    n = C.c_uint64()
    assert nat.lib.m40llm_context_launch_count(nat.ctx, C.byref(n)) == 0
    return int(n.value)


def workload_config(global_lens, world):
    """The `config` object both arms print: BASELINE.json configs[2], the configuration the metric is quoted on."""
    att = np.asarray(global_lens, np.int64) + 1
    per_gpu_bytes = layer_weight_bytes() + attention_bytes(att) // max(world, 1)
    return {"workload": "llama3-8b-shaped decode layer, batch 32 varlen [512,8192], q8_0 FFN (BASELINE configs[2])",
            "hidden": H, "q_heads": QH, "kv_heads": KVH, "head_dim": HD, "ffn": F, "batch_per_gpu": B,
            "global_batch": int(B * world), "context_sum": int(att.sum()),
            "parallelism": f"one global batch of {B * world} sequences dealt to {world} GPU(s), longest first, "
                           f"{B} per GPU; weights replicated; no collective",
            "l2": f"inputs larger than L2: about {per_gpu_bytes / 1e6:.0f} MB per GPU per step, {N_WEIGHT_SETS} weight "
                  "sets rotated"}


class CpuLayer:
    """Oracle layer over a bounded sample of the batch: the first `n_seq` sequences, caches built once."""

    def __init__(self, O, sets, x, lens, n_seq=8):
        self.O, self.sets, self.x, self.lens = O, sets, x, lens
        self.cfg = O.LayerCfg(H, QH, KVH, HD, F, 1, 0, EPS, THETA, 1.0)
        self.seqs = list(range(min(n_seq, len(lens))))
        self.caches = []
        for b in self.seqs:
            n = int(lens[b])
            k, v = kv_for_sequence(b, n)
            K = np.zeros((n + 1, KVH, HD), np.float16)
            V = np.zeros((n + 1, KVH, HD), np.float16)
            K[:n], V[:n] = k, v
            self.caches.append((K, V))

    def step(self, i):
        """One sequence's layer-step; returns seconds."""
        j = i % len(self.seqs)
        b = self.seqs[j]
        t0 = time.perf_counter()
        self.O.decode_layer(self.cfg, self.x[b], self.sets[0], self.caches[j][0], self.caches[j][1], int(self.lens[b]))
        return time.perf_counter() - t0

    def describe(self):
        c = [int(self.lens[b]) for b in self.seqs]
        return (f"oracle layer, one sequence per call, cycling the first {len(c)} of the {B} sequences (contexts "
                f"{min(c)}..{max(c)}); every call streams all {layer_weight_bytes() / 1e6:.0f} MB of layer weights for "
                f"one token, where the GPU arm reads them once per {B}-row step")


def parity_gate(nat, O, layer, kv, sets, x_rows, lens_rows, global_ids):
    """One eager step of this rank's batch against the oracle, outside every timed region: four rows (shortest and
    longest context and two more), layer output and the K/V rows the prologue appended. Returns the record for the
    bench line; raises SystemExit(3) on a miss."""
    rows = sorted({int(np.argmin(lens_rows)), int(np.argmax(lens_rows)), 7 % len(lens_rows), 20 % len(lens_rows)})
    layer.enqueue(0)
    nat.sync(1)
    out = layer.dout.download(np.float32, (layer.rows, H))
    cfg = O.LayerCfg(H, QH, KVH, HD, F, 1, 0, EPS, THETA, 1.0)
    worst, fails = 0.0, []
    for r in rows:
        n = int(lens_rows[r])
        k, v = kv_for_sequence(global_ids[r], n)
        K = np.zeros((n + 1, KVH, HD), np.float16)
        V = np.zeros((n + 1, KVH, HD), np.float16)
        K[:n], V[:n] = k, v
        eout, _, _ = O.decode_layer(cfg, x_rows[r], sets[0], K, V, n)
        kd, vd = np.zeros((KVH, HD), np.float16), np.zeros((KVH, HD), np.float16)
        rc = nat.lib.m40llm_kvcache_debug_read_token(nat.ctx, kv, r, n, kd.ctypes.data_as(C.c_void_p),
                                                     vd.ctypes.data_as(C.c_void_p))
        assert rc == 0, rc
        for name, got, exp in (("out", out[r], eout), ("k", kd.astype(np.float32), K[n].astype(np.float32)),
                               ("v", vd.astype(np.float32), V[n].astype(np.float32))):
            err = np.abs(got.astype(np.float64) - exp.astype(np.float64))
            excess = float(np.max(err - (ATOL + RTOL * np.abs(exp))))
            worst = max(worst, float(err.max()))
            if not np.all(np.isfinite(got)) or excess > 0:
                fails.append(f"row {r} (context {n}) {name}: max err {err.max():.3e}")
    st = np.zeros(1, np.uint32)
    assert nat.lib.m40llm_context_take_device_status(nat.ctx, st.ctypes.data) == 0
    if st[0] != 0:
        fails.append(f"device status word {int(st[0])}")
    if fails:
        sys.stderr.write("PARITY FAILED against the oracle, nothing timed: " + "; ".join(fails) + "\n")
        raise SystemExit(3)
    return {"checked": "layer output and appended K/V rows of one eager step vs the oracle layer, before any timing",
            "rows": rows, "contexts": [int(lens_rows[r]) for r in rows], "max_abs_err": worst,
            "tolerance": f"{ATOL} + {RTOL}*|e|", "passed": True}


def attention_only_case(nat, args):
    """The dominant kernel on a small batch (KV larger than L2, well under 1 GB on the device): the case the
    committed profiler summaries are taken on. Prints its own one-line summary, not the bench line."""
    n = args.attention_only
    lens = np.random.default_rng(0).integers(LMIN, LMAX + 1, size=B).astype(np.uint32)[:n]
    kv = nat.kv_dense(LMAX + 8, n, KVH, HD)
    for b in range(n):
        k, v = kv_for_sequence(b, int(lens[b]))
        nat.kv_fill(kv, b, k, v)
    layer = Layer(nat, kv, None, n)
    layer.dq.upload(np.random.default_rng(1).standard_normal((n, QH * HD), dtype=np.float32))
    layer.dids.upload(np.arange(n, dtype=np.uint32))
    layer.dlens.upload(lens)
    ev = Events(nat)
    for _ in range(3):
        layer.attention_only()
    nat.sync(1)
    ev.start()
    for _ in range(args.steps):
        layer.attention_only()
    ms = ev.stop_ms() / args.steps
    by = attention_bytes(lens)
    print(json.dumps({"case": "attention_only", "sequences": n, "context_sum": int(lens.sum()),
                      "algorithmic_bytes": by, "ms_per_launch": ms, "achieved_gbs": by / ms / 1e6}), flush=True)
    nat.lib.m40llm_kvcache_destroy(kv)


def ffn_only_case(nat, O, args):
    """The Q8_0 SwiGLU FFN of the bench layer alone (187 MB of weights per call, three weight sets rotated so that
    nothing survives in L2): the case the committed profiler summaries of the projection kernels are taken on."""
    rows = args.ffn_only
    rng = np.random.default_rng(3)
    sets = []
    for _ in range(3):
        w = {n: nat.buf(O.q80_quantize(rng.standard_normal(s, dtype=np.float32) * np.float32(0.02)))
             for n, s in dict(wg=(F, H), wu=(F, H), wd=(H, F)).items()}
        sets.append(w)
    dx = nat.buf(rng.standard_normal((rows, H), dtype=np.float32))
    dh, do = nat.buf(rows * F * 4), nat.buf(rows * H * 4)
    L, ctx = nat.lib, nat.ctx

    def call(i):
        w = sets[i % 3]
        rc = L.m40llm_ffn_swiglu_q80_f32_async(ctx, dx.ptr, w["wg"].ptr, w["wu"].ptr, w["wd"].ptr, None, dh.ptr, do.ptr,
                                               rows, H, F, 1)
        assert rc == 0, rc

    ev = Events(nat)
    for i in range(3):
        call(i)
    nat.sync(1)
    ev.start()
    for i in range(args.steps):
        call(i)
    ms = ev.stop_ms() / args.steps
    by = 3 * F * (H // 32) * 34
    print(json.dumps({"case": "ffn_only", "rows": rows, "algorithmic_bytes": by, "ms_per_call": ms,
                      "achieved_gbs": by / ms / 1e6}), flush=True)


def layer_only_case(nat, O, args):
    """The whole layer chain at `--layer-only ROWS` rows on a context of 7969 tokens per row (graph replays, two
    weight sets rotated): the case the committed launch lists of the one-row chain are taken on."""
    rows = args.layer_only
    _, sets, x = make_inputs(O, 1)
    dw = [{n: nat.buf(a) for n, a in w.items()} for w in sets]
    ctxlen = 7968
    kv = nat.kv_dense(ctxlen + 8, rows, KVH, HD)
    for b in range(rows):
        k, v = kv_for_sequence(b, ctxlen)
        nat.kv_fill(kv, b, k, v)
    layer = Layer(nat, kv, dw, rows)
    layer.dx.upload(x[:rows])
    layer.dids.upload(np.arange(rows, dtype=np.uint32))
    layer.dpos.upload(np.full(rows, ctxlen, np.uint32))
    layer.dlens.upload(np.full(rows, ctxlen + 1, np.uint32))
    for w in range(N_WEIGHT_SETS):
        layer.enqueue(w)
    nat.sync(1)
    graphs = [layer.capture(w) for w in range(N_WEIGHT_SETS)]
    ev = Events(nat)
    L, ctx = nat.lib, nat.ctx
    for i in range(3):
        assert L.m40llm_cuda_graph_launch(ctx, graphs[i % N_WEIGHT_SETS], 1) == 0
    nat.sync(1)
    ev.start()
    for i in range(args.steps):
        assert L.m40llm_cuda_graph_launch(ctx, graphs[i % N_WEIGHT_SETS], 1) == 0
    ms = ev.stop_ms() / args.steps
    by = step_bytes([ctxlen + 1] * rows)
    print(json.dumps({"case": "layer_only", "rows": rows, "context": ctxlen + 1, "algorithmic_bytes": by,
                      "ms_per_step": ms, "achieved_gbs": by / ms / 1e6}), flush=True)


def compressed_case(nat, ev, peak, calls=16, reps=20):
    """Long-context compressed attention (BASELINE configs[3] shape): Qwen2.5-3B heads, context 32768 in the FP16-K /
    q4-V cache, 512-token ring, 64-token blocks, top 64. Four caches rotate; `calls` calls are captured in ONE graph so
    that the timing is the device's, not the launch path's."""
    L, ctx = nat.lib, nat.ctx
    cq, ckv, chd, cL, cR, cbs, ctop = 16, 2, 128, 32768, 512, 64, 64
    crng = np.random.default_rng(7)
    caches = []
    for _ in range(4):
        c = nat.kv_compressed(cL, 1, ckv, chd, cR, cbs, ctop)
        nat.kv_fill(c, 0, crng.standard_normal((cL, ckv, chd), dtype=np.float32).astype(np.float16),
                    crng.standard_normal((cL, ckv, chd), dtype=np.float32).astype(np.float16), final_len=cL)
        caches.append(c)
    cdq = nat.buf(crng.standard_normal(cq * chd, dtype=np.float32))
    cdo = nat.buf(cq * chd * 4)
    f = L.m40llm_attention_last_token_f32_gqa_block_select_exact_fp16_k_q4_v_old_direct_async
    n0 = launches(nat)
    assert f(ctx, caches[0], 0, cdq.ptr, cq, cL, cR, cbs, ctop, cdo.ptr) == 0
    per_call = launches(nat) - n0
    for i in range(7):
        assert f(ctx, caches[i % 4], 0, cdq.ptr, cq, cL, cR, cbs, ctop, cdo.ptr) == 0
    nat.sync(1)
    assert L.m40llm_cuda_graph_begin_capture(ctx, 1) == 0
    for i in range(calls):
        assert f(ctx, caches[i % 4], 0, cdq.ptr, cq, cL, cR, cbs, ctop, cdo.ptr) == 0
    gexec = C.c_void_p()
    assert L.m40llm_cuda_graph_end_capture(ctx, 1, C.byref(gexec)) == 0 and gexec.value
    for i in range(3):
        assert L.m40llm_cuda_graph_launch(ctx, gexec, 1) == 0
    nat.sync(1)
    ev.start()
    for i in range(reps):
        assert L.m40llm_cuda_graph_launch(ctx, gexec, 1) == 0
    cms = ev.stop_ms() / (reps * calls)
    L.m40llm_cuda_graph_destroy(gexec)
    old_len = cL - cR
    # every old K once per kv head; selected q4 V + scales (<= top blocks per q head); the ring K and V
    cbytes = old_len * ckv * chd * 2 + cq * ctop * cbs * (chd // 2 + 4) + 2 * cR * ckv * chd * 2
    for c in caches:
        L.m40llm_kvcache_destroy(c)
    return {"ms_per_call": cms, "launches_per_call": per_call, "algorithmic_bytes": cbytes,
            "achieved_gbs": cbytes / (cms * 1e-3) / 1e9, "frac_of_hbm_peak": cbytes / (cms * 1e-3) / 1e9 / peak,
            "config": "16/2/128 heads, context 32768, ring 512, block 64, top 64"}


def splitk_case(nat, pkg, O, rank, world, dist, peak, reps=200, graphs=False):
    """One long sequence, split-K over the ranks (BASELINE configs[3]): Qwen2.5-3B heads (16 / 2 / 128), context 32768
    in the FP16-K / q4-V cache, 512-token ring, 64-token blocks, top 64. Every rank loads ONLY its own block range of
    old K / q4 V (the last rank also the ring); per call: local block scores -> local top-k pairs -> NCCL all-gather
    -> global top-k -> attention over the rank's selected blocks -> NCCL all-gather of the (m, l, o) triples -> merge,
    all enqueued on the decode stream with no host synchronisation. Also the whole Qwen-shaped layer around it
    (projections replicated on every rank, f16 weights, QKV bias, NeoX RoPE). Times are CUDA events on the decode
    stream, max over ranks. Rank 0 checks the attention output and the block lists against the oracle first."""
    import torch
    L_, ctx = nat.lib, nat.ctx
    splitk = pkg.splitk
    qh, kvh, hd, cL, cR, cbs, ctop, cH, cF = 16, 2, 128, 32768, 512, 64, 64, 2048, 11008
    rng = np.random.default_rng(7)
    k = rng.standard_normal((cL, kvh, hd), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((cL, kvh, hd), dtype=np.float32).astype(np.float16)
    q = rng.standard_normal(qh * hd, dtype=np.float32)
    old_len = cL - cR
    nb = (old_len + cbs - 1) // cbs
    b0, b1 = splitk.block_ranges(nb, world)[rank]
    t0, t1 = b0 * cbs, (cL if rank == world - 1 else min(b1 * cbs, old_len))
    kvc = nat.kv_compressed(cL + 8, 1, kvh, hd, cR, cbs, ctop)
    nat.kv_fill(kvc, 0, k[t0:t1], v[t0:t1], final_len=cL, tok_begin=t0)
    dev = torch.device("cuda", torch.cuda.current_device())
    dq = torch.from_numpy(q).to(dev)
    if world > 1:
        sk = splitk.DeviceSplitK(L_, ctx, kvc, dq, qh, hd, 0, cL)
        attend = lambda: sk.compressed(nb, ctop)
    else:
        dout = torch.empty(qh * hd, dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        f = L_.m40llm_attention_last_token_f32_gqa_block_select_exact_fp16_k_q4_v_old_direct_async

        def attend():
            rc = f(ctx, kvc, 0, C.c_void_p(dq.data_ptr()), qh, cL, cR, cbs, ctop, C.c_void_p(dout.data_ptr()))
            assert rc == 0, rc
            return dout, None
    torch.cuda.synchronize()
    out, blocks = attend()
    nat.sync(1)
    record = {"config": "16/2/128 heads, context 32768, ring 512, block 64, top 64; each rank holds only its block range",
              "ranks": world, "blocks_per_rank": [e - b for b, e in splitk.block_ranges(nb, world)]}
    if rank == 0:  # parity first
        old_k, q4, sc, rk, rv = O.compressed_state_from_dense(k, v, cL, cR)
        exp, esel, ecnt, _ = O.attention_compressed(old_k, q4, sc, rk, rv, q, qh, cL, cR, cbs, ctop)
        got = out.cpu().numpy()
        err = np.abs(got.astype(np.float64) - exp)
        if not np.all(err <= ATOL + RTOL * np.abs(exp)):
            sys.stderr.write(f"PARITY FAILED: split-K attention over {world} rank(s), max err {err.max():.3e}\n")
            raise SystemExit(3)
        record["parity"] = {"max_abs_err": float(err.max()), "passed": True}
        if blocks is not None:
            got_b = blocks.cpu().numpy().view(np.uint32)
            same = all(set(int(b) for b in got_b[h, :ctop]) == set(int(b) for b in esel[h, :ecnt[h]]) for h in range(qh))
            record["parity"]["block_lists_equal_oracle"] = bool(same)
    ev = Events(nat)
    for _ in range(5):
        attend()
    nat.sync(1)
    if dist is not None:
        dist.barrier()
    ev.start()
    for _ in range(reps):
        attend()
    att_ms = ev.stop_ms() / reps
    # the same chain (kernels + both all-gathers) captured once and replayed as one CUDA graph: no per-call host work
    graph_ms = None
    if world > 1 and graphs:
        replay = gout = None
        try:  # the capture itself runs nothing, so a rank that fails here does not leave the others in a collective
            replay, gout, _ = sk.capture_compressed(nb, ctop)
        except Exception as exc:  # capture of the collectives is not available on every torch / NCCL build
            record["attention_graph_error"] = f"{type(exc).__name__}: {exc}"[:200]
        okf = torch.tensor([1.0 if replay is not None else 0.0], device="cuda", dtype=torch.float64)
        dist.all_reduce(okf, op=dist.ReduceOp.MIN)
        if float(okf[0]) == 1.0:  # every rank holds a graph: replays are safe
            for _ in range(5):
                replay()
            nat.sync(1)
            record["attention_graph_equals_eager"] = bool(torch.equal(gout, out))
            dist.barrier()
            ev.start()
            for _ in range(reps):
                replay()
            graph_ms = ev.stop_ms() / reps
            nat.sync(1)

    # the whole layer around it: weights replicated; the step re-appends the last token (position cL - 1) on every
    # rank, so the block ranges stay those of the loaded data (the parity check above came first)
    host = pkg.host
    wr = np.random.default_rng(8)
    mk = lambda *sh: nat.buf((wr.standard_normal(sh, dtype=np.float32) * np.float32(0.02)).astype(np.float16))
    W = {"wq": mk(qh * hd, cH), "wk": mk(kvh * hd, cH), "wv": mk(kvh * hd, cH), "wo": mk(cH, qh * hd), "wg": mk(cF, cH),
         "wu": mk(cF, cH), "wd": mk(cH, cF)}
    Bq = nat.buf(wr.standard_normal(qh * hd, dtype=np.float32) * np.float32(0.02))
    Bk = nat.buf(wr.standard_normal(kvh * hd, dtype=np.float32) * np.float32(0.02))
    Bv = nat.buf(wr.standard_normal(kvh * hd, dtype=np.float32) * np.float32(0.02))
    ones = nat.buf(np.ones(cH, np.float32))
    dx = nat.buf(wr.standard_normal(cH, dtype=np.float32))
    dqb, datt = torch.empty(qh * hd, dtype=torch.float32, device=dev), torch.empty(qh * hd, dtype=torch.float32, device=dev)
    dx1, dhid, dlo = nat.buf(cH * 4), nat.buf(cF * 4), nat.buf(cH * 4)
    dids, dpos = nat.buf(np.array([0], np.uint32)), nat.buf(np.array([cL - 1], np.uint32))
    torch.cuda.synchronize()
    if world > 1:
        skl = splitk.DeviceSplitK(L_, ctx, kvc, dqb, qh, hd, 0, cL)

    def layer():
        rc = L_.m40llm_qkv_rmsnorm_rope_append_async(ctx, kvc, dx.ptr, ones.ptr, 1, EPS, W["wq"].ptr, W["wk"].ptr, W["wv"].ptr,
                                                    Bq.ptr, Bk.ptr, Bv.ptr, dids.ptr, dpos.ptr, 1, cH, qh, 1e6, 1.0, 1,
                                                    C.c_void_p(dqb.data_ptr()))
        assert rc == 0, rc
        if world > 1:
            o, _ = skl.compressed(nb, ctop)
            src = C.c_void_p(o.data_ptr())
        else:
            rc = L_.m40llm_attention_last_token_f32_gqa_block_select_exact_fp16_k_q4_v_old_direct_async(
                ctx, kvc, 0, C.c_void_p(dqb.data_ptr()), qh, cL, cR, cbs, ctop, C.c_void_p(datt.data_ptr()))
            assert rc == 0, rc
            src = C.c_void_p(datt.data_ptr())
        rc = L_.m40llm_attn_out_ffn_async(ctx, src, W["wo"].ptr, dx.ptr, ones.ptr, 1, EPS, W["wg"].ptr, W["wu"].ptr,
                                          W["wd"].ptr, 0, dx1.ptr, dhid.ptr, dlo.ptr, 1, cH, qh * hd, cF)
        assert rc == 0, rc

    for _ in range(5):
        layer()
    nat.sync(1)
    if dist is not None:
        dist.barrier()
    ev.start()
    for _ in range(reps):
        layer()
    layer_ms = ev.stop_ms() / reps
    nat.sync(1)
    layer_graph_ms = None
    if world > 1 and graphs:  # the whole layer step (prologue, split-K attention with its collectives, Wo + FFN) as one graph
        lreplay = None
        try:
            lreplay, _ = skl.capture(layer)
        except Exception as exc:
            record["layer_graph_error"] = f"{type(exc).__name__}: {exc}"[:200]
        okf = torch.tensor([1.0 if lreplay is not None else 0.0], device="cuda", dtype=torch.float64)
        dist.all_reduce(okf, op=dist.ReduceOp.MIN)
        if float(okf[0]) == 1.0:
            for _ in range(5):
                lreplay()
            nat.sync(1)
            dist.barrier()
            ev.start()
            for _ in range(reps):
                lreplay()
            lt = torch.tensor([ev.stop_ms() / reps], device="cuda", dtype=torch.float64)
            dist.all_reduce(lt, op=dist.ReduceOp.MAX)
            layer_graph_ms = float(lt[0])
            nat.sync(1)
            record["layer_graph_ms"] = layer_graph_ms
    st = np.zeros(1, np.uint32)
    assert L_.m40llm_context_take_device_status(ctx, st.ctypes.data) == 0 and st[0] == 0, int(st[0])
    if dist is not None:
        gflag = torch.tensor([0.0 if graph_ms is None else 1.0], device="cuda", dtype=torch.float64)
        dist.all_reduce(gflag, op=dist.ReduceOp.MIN)
        if float(gflag[0]) == 0.0:
            graph_ms = None
        else:
            gt = torch.tensor([graph_ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(gt, op=dist.ReduceOp.MAX)
            graph_ms = float(gt[0])
        t = torch.tensor([att_ms, layer_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        att_ms, layer_ms = float(t[0]), float(t[1])
    # per rank: its share of the old K (scoring), the selected q4 V + scales, the ring on the last rank
    cbytes = old_len * kvh * hd * 2 + qh * ctop * cbs * (hd // 2 + 4) + 2 * cR * kvh * hd * 2
    wbytes = sum(b.nbytes for b in W.values())
    if graph_ms is not None:
        record["attention_graph_ms"] = graph_ms
    record.update({"attention_ms": att_ms, "attention_calls_per_s": 1e3 / att_ms, "attention_algorithmic_bytes": cbytes,
                   "attention_frac_of_hbm_peak": cbytes / (att_ms * 1e-3) / 1e9 / (peak * world),
                   "layer_ms": layer_ms, "layer_tokens_per_s": 1e3 / layer_ms,
                   "layer_note": f"Qwen2.5-3B-shaped layer (hidden {cH}, FFN {cF}, f16 weights {wbytes / 1e6:.0f} MB replicated on "
                                 "every rank, QKV bias, NeoX RoPE theta 1e6), eager launches; only the attention shards",
                   "exchange": "none (one rank)" if world == 1 else
                               f"2 NCCL all-gathers per call on the decode stream: {qh * 64 * 8} B of top-k pairs and "
                               f"{qh * (hd + 2) * 4} B of triples per rank; selection and merge on the device"})
    L_.m40llm_kvcache_destroy(kvc)
    return record


def prefill_case(nat, ev, reps=10):
    """Packed varlen prefill attention (the tensor-bound sibling of the decode path): Llama-3-8B heads, four sequences
    of 2048, 1536, 1024 and 512 prompt tokens, causal, f32 in and out as the reference passes them. FLOPs counted
    algorithmically: 4 * head_dim per (q row, visible kv row, q head)."""
    L, ctx = nat.lib, nat.ctx
    qh, kvh, hd = QH, KVH, HD
    lens = np.array([2048, 1536, 1024, 512], np.uint32)
    off = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.uint32)
    rng = np.random.default_rng(17)
    total = int(lens.sum())
    dq = nat.buf(rng.standard_normal((total, qh, hd), dtype=np.float32))
    dk = nat.buf(rng.standard_normal((total, kvh, hd), dtype=np.float32))
    dv = nat.buf(rng.standard_normal((total, kvh, hd), dtype=np.float32))
    do = nat.buf(total * qh * hd * 4)
    dlen, doff = nat.buf(lens), nat.buf(off)
    call = lambda: L.m40llm_attention_prefill_f32_gqa_varlen_async(ctx, dq.ptr, dk.ptr, dv.ptr, doff.ptr, doff.ptr, dlen.ptr,
                                                                 dlen.ptr, len(lens), qh, kvh, hd, do.ptr)
    for _ in range(2):
        assert call() == 0
    nat.sync(0)
    e0, e1 = C.c_void_p(), C.c_void_p()
    assert L.m40llm_cuda_event_create(ctx, C.byref(e0)) == 0 and L.m40llm_cuda_event_create(ctx, C.byref(e1)) == 0
    assert L.m40llm_cuda_event_record(ctx, e0, 0) == 0
    for _ in range(reps):
        assert call() == 0
    assert L.m40llm_cuda_event_record(ctx, e1, 0) == 0
    ms = C.c_float()
    assert L.m40llm_cuda_event_elapsed_sync(ctx, e0, e1, C.byref(ms)) == 0
    ms = ms.value / reps
    pairs = float(sum(int(n) * (int(n) + 1) // 2 for n in lens))
    flops = 4.0 * hd * qh * pairs
    tf = flops / (ms * 1e-3) / 1e12
    peak_tf = 1636.2
    try:
        peak_tf = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        pass
    for b in (dq, dk, dv, do, dlen, doff):
        b.free()
    return {"prompt_tokens": total, "sequences": [int(n) for n in lens], "ms_per_call": ms, "prompt_tokens_per_s": total / (ms * 1e-3),
            "algorithmic_tflops": tf, "frac_of_bf16_tensor_peak": tf / peak_tf,
            "note": "mma.sync (legacy tensor path) flash-attention kernel over f16 copies of K / V made by a pack pass of the same call; "
                    "the call also reads the lengths back to the host as the reference does"}


def run_reference_arm(args, rank, world):
    """`--impl reference`: the reference's CPU path is Rust and cannot be built here (no cargo/rustc, no network),
    so the timed stand-in is the oracle port of that math, on all host threads. Rank 0 only. It is ONE CPU process on
    the box's host cores whatever --gpus says: its rate does not scale with the number of GPUs."""
    if rank != 0:
        return
    from oracle import oracle as O
    lens, sets, x = make_inputs(O, world)
    # torchrun exports OMP_NUM_THREADS=1; the reference arm is meant to use every host thread it can get
    O.set_num_threads(len(os.sched_getaffinity(0)))
    cores = O.num_threads()
    cpu = CpuLayer(O, sets, x, lens)
    times = []
    for i in range(args.warmup + args.steps):
        dt = cpu.step(i)
        if i >= args.warmup:
            times.append(dt)
    per_tok = float(np.mean(times))
    val = 1.0 / per_tok
    line = {
        "impl": "reference", "metric": "decode_layer_tokens_per_s", "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_tok * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(lens, world),
        "reference_scope": "one CPU process on the host cores of the box; the same rate at every --gpus",
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": cpu.describe() + ", one call per step, OpenMP over rows/heads"},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline line only: skip batch1, sweep, configs[1] and [3]")
    ap.add_argument("--ffn-only", type=int, default=0, metavar="ROWS",
                    help="small case for a profiler: the Q8_0 SwiGLU FFN alone for ROWS activation rows")
    ap.add_argument("--attention-only", type=int, default=0, metavar="N",
                    help="small case for a profiler: the batched attention call alone over the first N sequences")
    ap.add_argument("--layer-only", type=int, default=0, metavar="ROWS",
                    help="small case for a profiler: the layer chain at ROWS rows, context 7969")
    ap.add_argument("--compressed-only", action="store_true",
                    help="small case for a profiler: the 32K compressed attention call alone")
    ap.add_argument("--prefill-only", action="store_true",
                    help="small case for a profiler: the packed varlen prefill attention call alone")
    ap.add_argument("--workload", default="layer", choices=["layer", "splitk"],
                    help="layer: the batched decode layer (the contract's line); splitk: one 32K sequence, split-K over "
                         "the ranks (its own JSON line)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    from oracle import oracle as O  # input generation (Q8_0 quantiser), the parity gate and the cpu_baseline leg

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # the split-K exchange is two 8 KB all-gathers: plain rings
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pkg = load_package()
    nat = pkg.native.Native(pkg.native.lib(), device=local_rank)
    L, ctx = nat.lib, nat.ctx
    peak, peak_kind = measured_peak_gbs()

    if args.attention_only:
        attention_only_case(nat, args)
        return
    if args.ffn_only:
        ffn_only_case(nat, O, args)
        return
    if args.layer_only:
        layer_only_case(nat, O, args)
        return
    if args.compressed_only:
        print(json.dumps({"case": "compressed32k", **compressed_case(nat, Events(nat), peak, calls=4, reps=max(args.steps, 1))}),
              flush=True)
        return

    if args.prefill_only:
        print(json.dumps({"case": "prefill_varlen", **prefill_case(nat, Events(nat), reps=max(args.steps, 1))}), flush=True)
        return

    if args.workload == "splitk":
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        # this workload also replays the chain as CUDA graphs (kernels + NCCL all-gathers captured together)
        rec = splitk_case(nat, pkg, O, rank, world, dist, peak, graphs=True)
        if rank == 0:
            print(json.dumps({"metric": "splitk_attention_calls_per_s", "value": rec["attention_calls_per_s"], "unit": "calls/s",
                              "n_gpus": world, "higher_is_better": True, "scaling": "strong", "dtype": "f32",
                              "data": "synthetic", "config": {"workload": "qwen2.5-3b heads, one 32K sequence, compressed "
                                                              "cache, split-K (BASELINE configs[3])"}, **rec}), flush=True)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---------------- the global batch, dealt to the ranks (src/decode_batch.rs:143-286 builds the per-GPU plan)
    glens, sets, gx = make_inputs(O, world)
    shards = pkg.splitk.shard_sequences(glens, world, max_per_rank=B) if world > 1 else [list(range(B))]
    mine = shards[rank]
    lens, x = glens[mine], np.ascontiguousarray(gx[mine])
    dw = [{n: nat.buf(a) for n, a in w.items()} for w in sets]
    kv = nat.kv_dense(LMAX + 8, B, KVH, HD)
    for b in range(B):
        k, v = kv_for_sequence(mine[b], int(lens[b]))
        nat.kv_fill(kv, b, k, v)
    layer = Layer(nat, kv, dw, B)
    ids = np.arange(B, dtype=np.uint32)
    pos = lens.copy()          # the new token of sequence b sits at position lens[b]
    att_lens = lens + 1
    layer.dx.upload(x)
    layer.dids.upload(ids)
    layer.dpos.upload(pos)
    layer.dlens.upload(att_lens)

    # ---------------- parity gate (also the eager pass that sizes the scratch arenas), then one graph per weight set
    parity = parity_gate(nat, O, layer, kv, sets, x, lens, mine)
    for w in range(N_WEIGHT_SETS):
        layer.enqueue(w)
    nat.sync(1)
    graphs = [layer.capture(w) for w in range(N_WEIGHT_SETS)]
    ev = Events(nat)

    def barrier():
        nat.sync()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()

    def graph_block(i0):
        for i in range(i0, i0 + args.steps):
            assert L.m40llm_cuda_graph_launch(ctx, graphs[i % N_WEIGHT_SETS], 1) == 0

    # ---------------- device-resident timing
    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.wait_first_sample()
    for i in range(args.warmup):
        assert L.m40llm_cuda_graph_launch(ctx, graphs[i % N_WEIGHT_SETS], 1) == 0
    nat.sync(1)
    ev.start()
    graph_block(0)                      # pilot block (untimed for the result): sizes the number of timed blocks
    pilot_ms = ev.stop_ms()
    barrier()
    n0 = launches(nat)
    t_begin = sampler.mark()
    ms_step, blocks = timed_blocks(graph_block, ev, args.steps, pilot_ms)
    t_end = sampler.mark()
    barrier()
    clocks = sampler.stop(t_begin, t_end)
    # kernels per graph replay = kernels enqueued by one eager step
    n1 = launches(nat)
    layer.enqueue(0)
    nat.sync(1)
    per_step_launches = launches(nat) - n1
    ms_step_local = ms_step

    # the same loop without rotating the weight sets (what stays in the 126 MB L2 from one step to the next may hit)
    for i in range(3):
        assert L.m40llm_cuda_graph_launch(ctx, graphs[0], 1) == 0
    nat.sync(1)
    ev.start()
    wreps = max(args.steps, 20)
    for i in range(wreps):
        assert L.m40llm_cuda_graph_launch(ctx, graphs[0], 1) == 0
    ms_step_warm = ev.stop_ms() / wreps

    # ---------------- dominant kernel alone (batched decode attention), CUDA events on its stream
    for _ in range(3):
        layer.attention_only()
    nat.sync(1)
    # between timed launches the other sequences' KV (about 600 MB per pass) evicts any reuse: input > L2
    ev.start()
    for _ in range(20):
        layer.attention_only()
    apilot = ev.stop_ms()
    reps = max(20, int(np.ceil(MIN_TIMED_SECONDS * 1e3 / max(apilot / 20, 1e-3))))
    ev.start()
    for _ in range(reps):
        layer.attention_only()
    attn_ms = ev.stop_ms() / reps
    attn_bytes = attention_bytes(att_lens)
    attn_gbs = attn_bytes / (attn_ms * 1e-3) / 1e9

    # ---------------- end to end: the host-side layer driver (C++ mirror of the reference's batched layer forward)
    # with HOST buffers. Per step it uploads the batch plan and the activations from pinned memory, runs the layer
    # (graph replay after the first sight of a configuration), synchronises and copies the result back.
    host = pkg.host
    hl = host.DecodeLayer(ctx, host.LayerCfg(H, QH, KVH, HD, F, 0, EPS, THETA, 1.0), B)
    hw = []
    for d in dw:
        W = host.Weights()
        for n in ("attn_norm", "ffn_norm", "wq", "wk", "wv", "wo", "wg", "wu", "wd"):
            setattr(W, n, d[n].ptr)
        W.ffn_q80 = 1
        hw.append(W)
    kvcfg = host.dense_kv_cfg()
    hx = torch.from_numpy(x).pin_memory()
    hout = torch.empty((B, H), dtype=torch.float32).pin_memory()
    rid = np.arange(B, dtype=np.uint64)
    sid = ids.copy()
    kvl = att_lens.astype(np.uint32)
    act = np.ones(B, np.uint32)
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    h2d = hx.numel() * 4 + 3 * B * 4
    d2h = hout.numel() * 4

    def e2e_step(i):
        rc = hl.forward_host_raw(kv, hw[i % N_WEIGHT_SETS], kvcfg, B, vp(rid), vp(sid), vp(kvl), vp(act),
                                 C.c_void_p(hx.data_ptr()), C.c_void_p(hout.data_ptr()), True)
        assert rc == 0, (rc, host.last_error())

    for i in range(max(args.warmup, 2 * N_WEIGHT_SETS)):
        e2e_step(i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    e2e_pilot = time.perf_counter() - t0
    e2e_blocks = max(1, int(np.ceil(MIN_TIMED_SECONDS / max(e2e_pilot, 1e-6))))
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps * e2e_blocks):
        e2e_step(i)
    nat.sync()
    e2e_sync_s = (time.perf_counter() - t0) / (args.steps * e2e_blocks)
    # The same call in its two halves with TWO steps in flight (the host layer driver's begin / end): step i + 1's
    # upload and step i's download ride the prefill stream while the decode stream computes; every step still copies
    # its inputs in and its result out inside the timed region.
    hout2 = [torch.empty((B, H), dtype=torch.float32).pin_memory() for _ in range(2)]

    def e2e_begin(i):
        rc = hl.forward_host_begin_raw(i % 2, kv, hw[i % N_WEIGHT_SETS], kvcfg, B, vp(rid), vp(sid), vp(kvl), vp(act),
                                       C.c_void_p(hx.data_ptr()), True)
        assert rc == 0, (rc, host.last_error())

    def e2e_end(i):
        rc = hl.forward_host_end_raw(i % 2, C.c_void_p(hout2[i % 2].data_ptr()))
        assert rc == 0, (rc, host.last_error())

    def e2e_pipelined(n):
        e2e_begin(0)
        for i in range(n):
            if i + 1 < n:
                e2e_begin(i + 1)
            e2e_end(i)

    e2e_pipelined(max(args.warmup, 2 * N_WEIGHT_SETS) + 2)
    barrier()
    t0 = time.perf_counter()
    e2e_pipelined(args.steps * e2e_blocks)
    nat.sync()
    e2e_s = (time.perf_counter() - t0) / (args.steps * e2e_blocks)
    e2e_replays = hl.graph_replays()
    # the end-to-end call's result is the layer's: one more (untimed) call on weight set 0, the set whose eager step
    # the launch count above left in the device-resident output buffer
    e2e_step(0)
    e2e_err = float(np.max(np.abs(hout.numpy() - layer.dout.download(np.float32, (B, H)))))
    # and the two-in-flight form returns the same bytes as the one-call form (weight set 0 in both slots)
    for slot in range(2):
        assert hl.forward_host_begin_raw(slot, kv, hw[0], kvcfg, B, vp(rid), vp(sid), vp(kvl), vp(act),
                                         C.c_void_p(hx.data_ptr()), True) == 0
    for slot in range(2):
        assert hl.forward_host_end_raw(slot, C.c_void_p(hout2[slot].data_ptr())) == 0
        e2e_err = max(e2e_err, float(np.max(np.abs(hout2[slot].numpy() - hout.numpy()))))

    per_rank = None
    if dist is not None:
        t = torch.tensor([ms_step, e2e_s, e2e_sync_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, e2e_s, e2e_sync_s = float(t[0]), float(t[1]), float(t[2])
        mine_t = torch.tensor([ms_step_local, float(att_lens.sum()), attn_ms], device="cuda", dtype=torch.float64)
        allr = [torch.zeros_like(mine_t) for _ in range(world)]
        dist.all_gather(allr, mine_t)
        per_rank = [{"rank": r, "ms_per_step": float(a[0]), "context_sum": int(a[1]), "attention_ms": float(a[2])}
                    for r, a in enumerate(allr)]

    # ---------------- batch-1 step (the 70%-of-HBM target is stated on batch 1): own graph, rows = 1
    extra = {}
    if rank == 0 and not args.no_extras:
        l1 = Layer(nat, kv, dw, 1)
        l1.dx.upload(x[:1])
        longest = int(np.argmax(lens))
        l1.dids.upload(np.array([longest], np.uint32))
        l1.dpos.upload(np.array([lens[longest]], np.uint32))
        l1.dlens.upload(np.array([lens[longest] + 1], np.uint32))
        for w in range(N_WEIGHT_SETS):
            l1.enqueue(w)
        nat.sync(1)
        g1 = [l1.capture(w) for w in range(N_WEIGHT_SETS)]
        for i in range(5):
            assert L.m40llm_cuda_graph_launch(ctx, g1[i % N_WEIGHT_SETS], 1) == 0
        nat.sync(1)
        reps1 = max(args.steps, 2000)
        ev.start()
        for i in range(reps1):
            assert L.m40llm_cuda_graph_launch(ctx, g1[i % N_WEIGHT_SETS], 1) == 0
        ms1 = ev.stop_ms() / reps1
        b1 = step_bytes([lens[longest] + 1])
        extra["batch1"] = {"tokens_per_s": 1e3 / ms1, "ms_per_step": ms1, "context": int(lens[longest]) + 1,
                           "algorithmic_bytes": b1, "achieved_gbs": b1 / (ms1 * 1e-3) / 1e9,
                           "frac_of_hbm_peak": b1 / (ms1 * 1e-3) / 1e9 / peak, "peak_kind": peak_kind}

    # ---------------- batch sweep (BASELINE configs[4]): the same layer at 1 / 8 / 32 / 128 / 256 sequences with
    # contexts U[128, 16384], one graph per weight set. Cache contents do not matter for the time (zero-filled at
    # creation); lengths and positions are what the kernels read. With N > 1 the 32-, 128- and 256-sequence batches
    # are dealt to the ranks (strong scaling: the total work is fixed, the slowest rank sets the time).
    if not args.no_extras:
        sweep = []
        srng = np.random.default_rng(21)
        for sb in (1, 8, 32, 128, 256):
            slens_g = srng.integers(128, 16385, size=sb).astype(np.uint32)
            sx_g = srng.standard_normal((sb, H), dtype=np.float32)
            if world > 1 and sb < 32:
                continue
            sh = pkg.splitk.shard_sequences(slens_g, world, max_per_rank=(sb + world - 1) // world)[rank]
            slens, n_loc = slens_g[sh], len(sh)
            skv = nat.kv_dense(16384 + 8, n_loc, KVH, HD)
            sl = Layer(nat, skv, dw, n_loc)
            sl.dx.upload(sx_g[sh])
            sl.dids.upload(np.arange(n_loc, dtype=np.uint32))
            sl.dpos.upload(slens)
            sl.dlens.upload(slens + 1)
            for w in range(N_WEIGHT_SETS):
                sl.enqueue(w)
            nat.sync(1)
            sg = [sl.capture(w) for w in range(N_WEIGHT_SETS)]
            for i in range(4):
                assert L.m40llm_cuda_graph_launch(ctx, sg[i % N_WEIGHT_SETS], 1) == 0
            barrier()
            sreps = 200 if n_loc <= 32 else 60
            ev.start()
            for i in range(sreps):
                assert L.m40llm_cuda_graph_launch(ctx, sg[i % N_WEIGHT_SETS], 1) == 0
            sms = ev.stop_ms() / sreps
            sms_all = [sms]
            if dist is not None:
                t = torch.tensor([sms], device="cuda", dtype=torch.float64)
                allr = [torch.zeros_like(t) for _ in range(world)]
                dist.all_gather(allr, t)
                sms_all = [float(a[0]) for a in allr]
                sms = max(sms_all)
            # bytes the whole job moves per step: every GPU streams the weights, the KV is read once
            sbytes = step_bytes(slens_g + 1) + (world - 1) * layer_weight_bytes()
            sweep.append({"batch": sb, "context_sum": int(slens_g.sum()) + sb, "ms_per_step": sms,
                          "tokens_per_s": sb / (sms * 1e-3), "algorithmic_bytes": sbytes,
                          "frac_of_hbm_peak": sbytes / (sms * 1e-3) / 1e9 / (peak * world),
                          **({"ms_per_rank": sms_all} if world > 1 else {})})
            for sgraph in sg:
                L.m40llm_cuda_graph_destroy(sgraph)
            L.m40llm_kvcache_destroy(skv)
            for bname in ("dx", "dq", "datt", "dx1", "dx1n", "dhid", "dout", "dids", "dpos", "dlens"):
                getattr(sl, bname).free()
        if rank == 0:
            extra["batch_sweep" if world == 1 else "batch_sweep_strong_scaling"] = sweep

    if rank == 0 and not args.no_extras:
        extra["compressed32k"] = compressed_case(nat, ev, peak)
        extra["prefill_varlen"] = prefill_case(nat, ev)

    # ---------------- one long sequence, split-K over the ranks (BASELINE configs[3]); every rank takes part
    if not args.no_extras:
        sk_rec = splitk_case(nat, pkg, O, rank, world, dist, peak)
        if rank == 0:
            extra["splitk"] = sk_rec

    # ---------------- whole-model greedy decode at BASELINE configs[1] (TinyLlama-1.1B shape, batch 1, context 2048):
    # 22 distinct random f16 layers + lm_head, one CUDA graph per token step, ids chosen on the device.
    if rank == 0 and not args.no_extras:
        tH, tQ, tKV, tHD, tF, tV, tL, tCTX, tSTEPS = 2048, 32, 4, 64, 5632, 32000, 22, 2048, 96
        g = torch.Generator(device="cuda")
        g.manual_seed(11)
        keep = []

        def rnd(*shape, std=0.02):
            t = (torch.randn(*shape, generator=g, device="cuda", dtype=torch.float32) * std).to(torch.float16)
            keep.append(t)
            return t.data_ptr()

        ones = torch.ones(tH, device="cuda", dtype=torch.float32)
        lw = []
        for _ in range(tL):
            W = host.Weights()
            W.attn_norm = W.ffn_norm = ones.data_ptr()
            W.wq, W.wk, W.wv, W.wo = rnd(tQ * tHD, tH), rnd(tKV * tHD, tH), rnd(tKV * tHD, tH), rnd(tH, tQ * tHD)
            W.wg, W.wu, W.wd = rnd(tF, tH), rnd(tF, tH), rnd(tH, tF)
            W.ffn_q80 = 0
            lw.append(W)
        thead = host.ModelHead(rnd(tV, tH, std=0.5), ones.data_ptr(), rnd(tV, tH), tV)
        torch.cuda.synchronize()
        tkv = nat.kv_dense(tCTX + 3 * tSTEPS + 8, tL, tKV, tHD)
        trng = np.random.default_rng(5)
        for l in range(tL):
            k, v = (trng.standard_normal((tCTX, tKV, tHD), dtype=np.float32).astype(np.float16) for _ in range(2))
            nat.kv_fill(tkv, l, k, v)
        tm = host.DecodeModel(ctx, host.LayerCfg(tH, tQ, tKV, tHD, tF, 0, EPS, 1e4, 1.0), lw, thead, tkv, 1)
        tm.begin([17], [tCTX])
        tm.generate(4, use_graph=True, want_ids=False)            # eager step + capture + first replays
        nat.sync()
        t0 = time.perf_counter()
        tm.generate(tSTEPS, use_graph=True)
        tm.generate(tSTEPS, use_graph=True)
        t_tok = (time.perf_counter() - t0) / (2 * tSTEPS)
        tbytes = tL * ((2 * tQ * tHD * tH + 2 * tKV * tHD * tH + 3 * tF * tH) * 2 + 2 * (tCTX + tSTEPS) * tKV * tHD * 2) + tV * tH * 2
        extra["tinyllama_c1"] = {"tokens_per_s": 1.0 / t_tok, "ms_per_token": t_tok * 1e3, "layers": tL, "context": tCTX,
                                 "steps": 2 * tSTEPS, "graph_replays": tm.graph_replays(),
                                 "launches_per_token": tm.launches_per_step(), "algorithmic_bytes_per_token": tbytes,
                                 "achieved_gbs": tbytes / t_tok / 1e9, "frac_of_hbm_peak": tbytes / t_tok / 1e9 / peak,
                                 "timing": "wall clock around two generate calls (graph replays back to back, one "
                                           "device-to-host read of the ids at the end of each)"}
        tm.close()
        L.m40llm_kvcache_destroy(tkv)
        del keep

    # ---------------- CPU baseline (rank 0, N = 1): the oracle on a bounded sample of this batch
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        O.set_num_threads(len(os.sched_getaffinity(0)))
        cl = CpuLayer(O, sets, gx, glens)
        cl.step(0)
        spent, n = 0.0, 0
        while spent < CPU_BASELINE_SECONDS:
            spent += cl.step(n)
            n += 1
        cpu = {"value": n / spent, "unit": "tokens/s", "cores": O.num_threads(), "kind": "port",
               "sample": cl.describe() + f", {n} calls in {spent:.1f} s"}

    if dist is not None:
        ok = torch.tensor([1.0 if parity["passed"] else 0.0, parity["max_abs_err"]], device="cuda", dtype=torch.float64)
        dist.all_reduce(ok, op=dist.ReduceOp.MAX)
        parity["max_abs_err_all_ranks"] = float(ok[1])

    if rank == 0:
        # whole-job bytes per step: every GPU streams its own copy of the weights plus its sequences' KV
        sb = step_bytes(glens + 1) + (world - 1) * layer_weight_bytes()
        sb0 = step_bytes(att_lens)
        line = {
            "metric": "decode_layer_tokens_per_s", "value": world * B / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "timed_steps": blocks * args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": workload_config(glens, world),
            "parity": parity,
            "step_algorithmic_bytes": sb, "step_achieved_gbs": sb / (ms_step * 1e-3) / 1e9,
            "step_frac_of_hbm_peak": sb / (ms_step * 1e-3) / 1e9 / (peak * world),
            "warm_l2": {"ms_per_step": ms_step_warm, "step_frac_of_hbm_peak": sb0 / (ms_step_warm * 1e-3) / 1e9 / peak,
                        "note": "rank 0, one weight set replayed back to back (no rotation); the headline rotates "
                                f"{N_WEIGHT_SETS} sets so that no weight byte is reused from L2"},
            "roofline": {"kernel": "batched decode attention (attention + split merge), rank 0's sequences",
                         "bound": "hbm", "achieved": attn_gbs, "peak": peak, "unit": "GB/s", "frac": attn_gbs / peak,
                         "peak_kind": f"of {peak_kind}", "algorithmic_bytes": attn_bytes, "ms_per_launch": attn_ms,
                         "launches_timed": reps,
                         "traffic": None if NCU_TRAFFIC_RATIO is None else NCU_TRAFFIC_RATIO * attn_bytes},
            "e2e": {"value": world * B / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "in_flight": 2, "one_call_at_a_time": world * B / e2e_sync_s,
                    "graph_replays": e2e_replays, "timed_steps": args.steps * e2e_blocks,
                    "max_abs_diff_vs_device_resident_step": e2e_err},
            "gpu_launches": per_step_launches * args.steps * blocks,
            "launches_per_step": per_step_launches,
            "clocks": clocks,
        }
        if per_rank is not None:
            line["per_rank"] = per_rank
        line.update(extra)
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    hl.close()
    for g in graphs:
        L.m40llm_cuda_graph_destroy(g)
    L.m40llm_kvcache_destroy(kv)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
