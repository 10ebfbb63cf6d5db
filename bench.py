#!/usr/bin/env python
"""bench.py — decode tok/s of the sharded transformer-block forward path (BASELINE.json's metric):
Llama-3-8B bf16, bs=1, 2k context, layers sharded over N GPUs of one box (N=1 -> all local).

    python bench.py [--gpus N] [--steps K] [--warmup W]          # this repo's CUDA path
    python bench.py --impl reference [...]                        # the reference's CPU path (oracle port)
    torchrun --nproc-per-node N bench.py --gpus N ...             # N > 1, one rank per GPU
    python bench.py --model 70b [--gpus N]                        # BASELINE configs[3] as the main line
    python bench.py --workload prefill                            # BASELINE configs[4] as the main line
    python bench.py --workload nigenex [--sizes 2k,4k,4k-hd64]    # the Nigenex design beside the closest existing block
    python bench.py --workload setodra [--sizes 1k,2k]            # the Setodra design beside the closest existing model
    python bench.py --workload nuvarax [--sizes 1k,2k]            # the Nuvarax design beside the closest existing model
    python bench.py --workload netolorn [--sizes 1k,2k]           # the Netolorn design beside the closest existing models

A "step" is one decoded token: one pass of the hot path (embed -> blocks -> ln_f/lm_head/argmax) at batch 1.
tok/s follows the reference's definition (master.rs:131-166): prefill excluded.  Prints ONE JSON line (rank 0).

Timing: ONE enqueue of W + K graph replays per rank with a CUDA event after the W-th replay and after the last
(no barrier between warm-up and the timed region), CUDA events on the library's stream, barrier + synchronize on
both sides of the whole run, max over ranks.  Each token streams ~15 GB of weights, far beyond the 126 MB L2, so no
explicit L2 flush is needed between steps (stated in config.l2).

Besides the headline metric the line carries (N = 1 unless noted):
  parity     the first decoded tokens / logits of this very model checked against the oracle (every N), and the
             sha256 of all W+K greedy tokens — identical for every N because the kernels are order-deterministic
  config0    BASELINE configs[0]: Qwen3-0.6B (f16) greedy 32 tokens, GPU tok/s beside the oracle port on the host
  config3    BASELINE configs[3]: Llama-3-70B bf16 sharded over the 8 GPUs (only when N = 8, or --model 70b);
             config3_one_gpu at N = 1: the same model on ONE B200 (139 GB of weights fit its 180 GB)
  config4    BASELINE configs[4]: Llama-3-8B bs=32 x 4096 prefill with its own tensor-bound roofline object
"""
from __future__ import annotations

import argparse
import gc
import hashlib
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _cpu_plan():
    """Host threads for the CPU legs: the physical cores of ONE socket that this process may use, capped by the
    container's CPU quota.  (Round 1: the same 32 threads gave 4.5-9.1 tok/s run to run — threads and first-touch
    pages spread over two sockets and their SMT siblings.)"""
    allowed = sorted(os.sched_getaffinity(0))
    cores, seen = [], set()
    for c in allowed:
        try:
            base = f"/sys/devices/system/cpu/cpu{c}/topology/"
            pkg = int(open(base + "physical_package_id").read())
            cid = int(open(base + "core_id").read())
        except Exception:
            pkg, cid = 0, c
        if (pkg, cid) not in seen:
            seen.add((pkg, cid))
            cores.append((pkg, c))
    pk0 = min(p for p, _ in cores)
    sock = [c for p, c in cores if p == pk0]
    quota = len(allowed)
    try:
        q, per = open("/sys/fs/cgroup/cpu.max").read().split()
        if q != "max":
            quota = max(1, int(int(q) / int(per)))
    except Exception:
        pass
    n = max(1, min(len(sock), quota))
    return sock[:n], {"logical_cores": len(allowed), "physical_cores_socket0": len(sock), "cpu_quota_cores": quota}


CPU_SET, CPU_PLAN = _cpu_plan()
NCORES = len(os.sched_getaffinity(0))
# Before numpy/torch load an OpenMP runtime: bind the oracle's OpenMP threads 1:1 to those cores.
os.environ.setdefault("OMP_PROC_BIND", "true")
os.environ.setdefault("OMP_WAIT_POLICY", "passive")
os.environ.setdefault("OMP_NUM_THREADS", str(len(CPU_SET)))
os.environ.setdefault("GOMP_CPU_AFFINITY", " ".join(str(c) for c in CPU_SET))

E2E_WARM = 8  # untimed host-stepped steps before the timed ones (first replays of a freshly instantiated graph on every rank)
CTX_LEN = 2048
FIRST_TOKEN = 17
KV_SEED = 7
N_PARITY = 2


def model_config(name: str, max_seq: int):
    from cake_b200.config import llama3_70b, llama3_8b
    return {"8b": llama3_8b, "70b": llama3_70b}[name](max_seq=max_seq)


MODEL_LABEL = {"8b": "Llama-3-8B", "70b": "Llama-3-70B"}


def metric_name(model: str) -> str:
    return f"decode tok/s ({MODEL_LABEL[model]} bf16, bs=1, 2k ctx)"


def bytes_per_token(cfg, L: float, es: int = 2) -> float:
    """weights + lm_head + norms + embed row + KV read (length L) + KV write."""
    H, I, nh, nkv, hd, nl, V = (cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads,
                                cfg.num_key_value_heads, cfg.hd, cfg.num_hidden_layers, cfg.vocab_size)
    per_layer = H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * I + 2 * H
    w = nl * es * per_layer + es * V * H + es * H + es * H
    kv = nl * 2 * nkv * hd * es * L + nl * 2 * nkv * hd * es
    return float(w + kv)


def layer_bytes(cfg, L: float, es: int = 2) -> float:
    H, I = cfg.hidden_size, cfg.intermediate_size
    return float(es * (H * (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.hd + cfg.num_attention_heads * cfg.hd * H
                       + 3 * H * I + 2 * H) + 2 * es * cfg.num_key_value_heads * cfg.hd * (L + 1))


def head_bytes(cfg, es: int = 2) -> float:
    return float(es * cfg.vocab_size * cfg.hidden_size + 2 * es * cfg.hidden_size)


def peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm": float(d["hbm_gbs"]), "tc": float(d.get("bf16_tflops_sustained", 1459.3)),
                "tc_burst": float(d.get("bf16_tflops", 1701.1)), "src": "measured (MEASURED_PEAKS.json)"}
    return {"hbm": 6650.0, "tc": 1459.3, "tc_burst": 1701.1, "src": "fallback (B200_PROFILING.md)"}


class ClockSampler:
    """SM clock + throttle reasons sampled in-process through NVML every 10 ms.  NVML is initialised when the
    sampler is created — long before any timed region; round 1 forked `nvidia-smi` right before the timed steps and
    its driver-wide initialisation (all GPUs of the box) stalled one step of every leg by 10-50 ms."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, device: int):
        self.rows, self.on, self.h, self.err = [], False, None, None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            idx = device
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                try:
                    idx = int(vis.split(",")[device])
                except Exception:
                    idx = device
            self.h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.t = threading.Thread(target=self._loop, daemon=True)
            self.alive = True
            self.t.start()
        except Exception as e:  # noqa: BLE001
            self.err = str(e)

    def _loop(self):
        nv = self.nv
        while self.alive:
            if self.on:
                try:
                    sm = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                    try:
                        rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                    except Exception:
                        rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                    self.rows.append((float(sm), int(rs)))
                except Exception:
                    pass
            time.sleep(0.01)

    def start(self):
        self.rows, self.on = [], True

    def stop(self) -> dict:
        self.on = False
        if self.h is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [f"nvml unavailable: {self.err}"], "samples": 0}
        sm = [r[0] for r in self.rows]
        reasons = set()
        for _, rs in self.rows:
            for bit, name in self.REASONS.items():
                if rs & bit:
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_sm, "reasons": sorted(reasons),
                "samples": len(sm), "period_ms": 10, "how": "pynvml in-process, sampled only while the timed region runs"}

    def close(self):
        self.alive = False


# ------------------------------------------------------------------------------------------------
def host_info() -> dict:
    model = ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    model = line.split(":", 1)[1].strip()
                    break
    except Exception:
        pass
    return {"cpu": model, **CPU_PLAN, "threads_used": len(CPU_SET)}


def oracle_threads() -> int:
    from oracle import oracle as O
    O.lib().ora_set_num_threads(len(CPU_SET))
    return O.lib().ora_num_threads()


def time_oracle_tokens(om, cache, x_or_tok, pos0: int, n_tokens: int, budget_s: float, scale: float = 1.0) -> dict:
    """Times `n_tokens` decode tokens of an OracleModel (embed -> all its layers -> ln_f/lm_head -> argmax)."""
    from oracle import oracle as O
    times, toks, logits = [], [], []
    tok = x_or_tok
    spent = 0.0
    for i in range(n_tokens):
        t0 = time.perf_counter()
        lg = om.forward([tok], pos0 + i, cache)
        nt = O.argmax(lg)
        dt = time.perf_counter() - t0
        times.append(dt)
        toks.append(nt)
        logits.append(lg)
        tok = nt
        spent += dt
        if spent > budget_s and i >= 1:
            break
    return {"times": times, "tokens": toks, "logits": logits}


def cpu_reference_tok_s(cfg, n_tokens: int, budget_s: float, layers_cap=None) -> dict:
    """The reference's CPU path (oracle port, host threads of one socket) on the same workload: bs=1 decode at KV
    length CTX_LEN.  Bounded sample: `n_tokens` tokens over `n_sample` of the layers (+ the full ln_f/lm_head
    tail), scaled to the whole model — per-layer work is identical across layers.  Used by --impl reference, which
    must not touch the GPU; the N=1 CUDA arm times the oracle on the real 32-layer model instead (see parity_leg)."""
    import numpy as np
    from cake_b200.synth import make_head, make_layer
    from oracle import oracle as O

    nthreads = oracle_threads()
    t_build = time.perf_counter()
    nl = cfg.num_hidden_layers
    n_sample = min(nl, layers_cap or nl)
    # one random layer + distinct-memory clones: CPU timing is data independent; avoids minutes of host RNG
    base = make_layer(cfg, 0, "bf16", seed=1234)
    sd = make_head(cfg, "bf16", seed=1234)
    for i in range(n_sample):
        for k, v in base.items():
            sd[k.replace(".layers.0.", f".layers.{i}.")] = v if i == 0 else v.clone()
    om = O.OracleModel(cfg, sd, "bf16", max_seq=CTX_LEN + 64, layers=range(n_sample))
    cache = om.new_cache(CTX_LEN + 64)
    rng = np.random.default_rng(0)
    for l in range(n_sample):
        k, v = cache.kv(l)
        k[:, :CTX_LEN] = O.round_to(rng.standard_normal((k.shape[0], CTX_LEN, k.shape[2]), dtype=np.float32), "bf16")
        v[:, :CTX_LEN] = k[:, :CTX_LEN]
        cache.set_len(l, CTX_LEN)
    x = om.embed([FIRST_TOKEN])
    build_s = time.perf_counter() - t_build

    def one_token(pos):
        t0 = time.perf_counter()
        h = om.forward_layers(x, 0, n_sample, pos, cache)
        t1 = time.perf_counter()
        lg = om.logits(h)
        O.argmax(lg)
        t2 = time.perf_counter()
        return t1 - t0, t2 - t1

    one_token(CTX_LEN)  # warm-up (page-in)
    tl, th = [], []
    spent = 0.0
    for i in range(n_tokens):
        a, b = one_token(CTX_LEN + 1 + i)
        tl.append(a)
        th.append(b)
        spent += a + b
        if spent > budget_s and i >= 1:
            break
    per_tok = [a * nl / n_sample + b for a, b in zip(tl, th)]
    t_tok = statistics.mean(per_tok)
    return {"value": 1.0 / t_tok, "unit": "tok/s", "cores": nthreads, "kind": "port",
            "sample": f"{len(tl)} decode tokens at KV length {CTX_LEN}, {n_sample}/{nl} layers timed and scaled + full lm_head "
                      f"(oracle/cake_oracle.c, OpenMP bound to the physical cores of one socket; setup {build_s:.0f}s untimed)",
            "spread_tok_s": {"min": 1.0 / max(per_tok), "median": 1.0 / statistics.median(per_tok), "max": 1.0 / min(per_tok)},
            "ms_per_token": t_tok * 1e3, "host": host_info()}


def run_reference(args):
    """--impl reference: the reference's own CPU implementation cannot be built (Rust, no toolchain);
    the oracle port stands in, timed on this box's host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = model_config(args.model, 4096)
    steps, warm = args.steps, args.warmup
    # keep the whole run within a few minutes: first probe 4 layers, then size the sample
    probe = cpu_reference_tok_s(cfg, 1, 5.0, layers_cap=4)
    est_full = probe["ms_per_token"] / 1e3
    budget = 150.0
    nl = cfg.num_hidden_layers
    cap = nl if est_full * (steps + warm) <= budget else max(2, int(nl * budget / (est_full * (steps + warm))))
    if args.model == "70b":
        cap = min(cap, 8)  # 1.7 GB per layer on the host
    res = cpu_reference_tok_s(cfg, steps, budget, layers_cap=cap)
    line = {
        "impl": "reference", "metric": metric_name(args.model), "value": res["value"], "unit": "tok/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": res["ms_per_token"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{MODEL_LABEL[args.model]} bf16, 1 process, bs=1 decode, 2k context, CPU (reference path: oracle port)",
                   "kv_len": CTX_LEN, "reference_binary": "unbuildable here (Rust; no cargo/rustc) -> oracle port"},
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample", "spread_tok_s")},
        "e2e": {"value": res["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "host": res["host"],
    }
    emit(line)


# ------------------------------------------------------------------------------------------------
class Env:
    """Process-wide state of the CUDA arm: rank / world, torch.distributed, the clock sampler."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and args.gpus > 1 and self.world == 1:
            raise SystemExit("launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
        torch.cuda.set_device(self.local)
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner off stdout: rank 0 prints exactly one JSON line
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device(f"cuda:{self.local}"))
        self.sampler = ClockSampler(self.local) if self.rank == 0 else None
        self.dev = f"cuda:{self.local}"

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = self.torch.tensor([v], device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def gather(self, obj):
        if self.world == 1:
            return [obj]
        out = [None] * self.world
        self.dist.all_gather_object(out, obj)
        return out


class Shard:
    """One rank's share of a decode job: ctx, its blocks (rank 0: + head), the KV cache, the decode graph."""

    def __init__(self, env: Env, model: str, cache_cap: int, keep_host: bool):
        import torch
        from cake_b200.model import Cache, Context, TextModelBase
        from cake_b200.synth import LazyCheckpoint
        self.env, self.model_name = env, model
        self.cfg = cfg = model_config(model, 4096)
        self.sd = LazyCheckpoint(cfg, "bf16", seed=1234, device=env.dev, host_copy=keep_host)
        self.ctx = Context(cfg, self.sd, "bf16", device=env.local, max_seq=4096)
        self.ctx.cache = Cache(self.ctx, 1, cache_cap)
        self.cache_cap = cache_cap
        if env.world == 1:
            self.tm = TextModelBase.load(self.ctx)
            self.blocks, self.idx = self.tm.blocks, list(range(cfg.num_hidden_layers))
        else:
            from cake_b200.parallel import ShardedMaster, Worker, init_comm
            init_comm(self.ctx, env.rank, env.world)
            if env.rank == 0:
                self.master = ShardedMaster(self.ctx, env.world)
                self.tm = self.master.model
                self.blocks, self.idx = self.master.local, self.master.local_idx
            else:
                self.worker = Worker(self.ctx, env.rank, env.world)
                self.blocks, self.idx = self.worker.block_list()
        self.sd.drop_layers()
        self.sd.drop_head()
        torch.cuda.empty_cache()
        self.pos = 0
        self.built = False

    # -- C ABI calls, identical on every rank
    def fill(self, length: int):
        self.ctx.cache.clear()
        self.ctx.cache.fill_synthetic(self.idx, length, KV_SEED)   # KV cache at 2k context (prefill is outside the metric)
        self.ctx.sync()
        self.pos = length

    def build(self):
        from cake_b200.capi import check, int_array, lib, ptr_array
        check(lib().cake_b200_decode_build(self.ctx.h, ptr_array([b.h for b in self.blocks]), int_array(self.idx), len(self.blocks),
                                           self.ctx.cache.h, self.env.rank, self.env.world))
        self.built = True

    def begin(self, first: int):
        from cake_b200.capi import check, lib
        check(lib().cake_b200_decode_begin(self.ctx.h, first if self.env.rank == 0 else 0, self.pos))

    def run(self, n: int):
        from cake_b200.capi import check, lib
        check(lib().cake_b200_decode_run(self.ctx.h, n))
        self.pos += n

    def event(self):
        e = self.env.torch.cuda.Event(enable_timing=True)
        e.record(self.ctx.torch_stream)
        return e

    def wait(self, ev):
        if self.env.rank == 0:
            ev.synchronize()
        else:
            # sleep-poll instead of a spinning wait: N-1 worker processes spinning next to rank 0's per-token sync
            # starve it when the container's CPU quota is below the visible core count
            while not ev.query():
                time.sleep(0.0005)

    def tokens(self, n: int):
        from cake_b200.capi import c_uint32, check, lib
        out = (c_uint32 * n)()
        check(lib().cake_b200_decode_tokens(self.ctx.h, out, n))
        return [int(t) for t in out]

    def step_trace(self, n: int):
        """Per-step %globaltimer stamps of the decode kernels of this rank (CTA 0): entry / input acquired / exit."""
        import ctypes
        from cake_b200.capi import lib
        buf = (ctypes.c_uint64 * (8 * n))()
        if not hasattr(lib(), "cake_b200_decode_trace") or lib().cake_b200_decode_trace(self.ctx.h, buf, n) != 0:
            return None
        return [list(buf[8 * i:8 * i + 8]) for i in range(n)]

    def close(self):
        self.ctx.close()
        self.env.torch.cuda.empty_cache()


def decode_leg(env: Env, model: str, K: int, W: int, n_e2e: int, parity: bool, isolated: bool, cpu_leg: bool) -> dict:
    """The headline measurement for `model` over env.world GPUs.  Every rank calls this; rank 0 returns the result."""
    import torch
    from cake_b200.capi import byref, c_uint32, check, lib
    world, rank = env.world, env.rank
    cache_cap = CTX_LEN + K + W + n_e2e + E2E_WARM + 64
    sh = Shard(env, model, cache_cap, keep_host=(parity and rank == 0))
    cfg = sh.cfg
    sh.fill(CTX_LEN)
    sh.build()

    # ---- device-timed leg: W warm-up + K timed replays in ONE enqueue ------------------------------------------
    sh.begin(FIRST_TOKEN)
    env.barrier()
    sh.ctx.sync()
    l0 = sh.ctx.launch_count()
    sh.run(W)                                             # warm-up steps (untimed)
    e0 = sh.event()
    if env.sampler:
        env.sampler.start()
    sh.run(K)                                             # EXACTLY K timed steps
    e1 = sh.event()
    sh.wait(e1)
    clocks = env.sampler.stop() if env.sampler else None
    ms = e0.elapsed_time(e1)
    launches = (sh.ctx.launch_count() - l0) * K // (W + K)
    env.barrier()
    ms_all = env.max_over_ranks(ms)
    all_tokens = sh.tokens(W + K) if rank == 0 else None
    trace = sh.step_trace(K)
    traces = env.gather(trace)

    # ---- e2e: one token per call through the public API with HOST buffers (token id H2D, token D2H, sync) ---------
    lat = []
    if n_e2e > 0:
        tok = all_tokens[-1] if rank == 0 else 0
        sh.begin(tok)
        # a generation-2 collection of this process's heap (torch + numpy + the checkpoint dicts: ~1M tracked objects) takes
        # tens of ms and lands on whichever step trips the counter — the N=4 rehearsal showed exactly one 70 ms step in 64
        # (p50 3.00 ms): collect now, keep the collector off while steps are being timed with the host clock
        gc.collect()
        gc.disable()
        env.barrier()
        if rank == 0:
            nxt = c_uint32()
            cur = tok
            for _ in range(E2E_WARM):  # untimed warm-up of the host-stepped path
                check(lib().cake_b200_decode_step_host(sh.ctx.h, cur, byref(nxt)))
                cur = nxt.value
            t0 = time.perf_counter()
            for _ in range(n_e2e):     # workers (N>1) have pre-enqueued the same number of replays
                t1 = time.perf_counter()
                check(lib().cake_b200_decode_step_host(sh.ctx.h, cur, byref(nxt)))
                cur = nxt.value
                lat.append(time.perf_counter() - t1)
            e2e_s = time.perf_counter() - t0
            sh.pos += n_e2e + E2E_WARM
        else:
            sh.run(n_e2e + E2E_WARM)
            sh.wait(sh.event())
        gc.enable()
        env.barrier()

    # ---- parity: the first tokens of this very model against the oracle, teacher-forced (rank 0 checks) ----------
    par = None
    if parity:
        par = parity_leg(env, sh, all_tokens, cpu_leg)

    if rank != 0:
        sh.close()
        return {}

    # ---- assemble ----------------------------------------------------------------------------------------------
    pk = peaks()
    tok_s = K / (ms_all / 1e3)
    L_mean = CTX_LEN + W + K / 2.0
    bpt = bytes_per_token(cfg, L_mean)
    n_local = len(sh.idx)
    launch_bytes = n_local * layer_bytes(cfg, L_mean) + head_bytes(cfg)   # rank 0's kernels: its layers + ln_f/lm_head/embed row
    launch_ms = ms_all / K
    G = cfg.num_attention_heads // cfg.num_key_value_heads
    roof = {"bound": "hbm", "kernel": f"decode_mega_kernel<bf16,{cfg.hd},{G}> (all local layers + ln_f + lm_head + argmax)",
            "achieved": round(launch_bytes / (launch_ms * 1e-3) / 1e9, 1), "peak": pk["hbm"], "unit": "GB/s",
            "frac": round(launch_bytes / (launch_ms * 1e-3) / 1e9 / pk["hbm"], 4),
            "traffic": TRAFFIC_NCU["bytes"] if (world == 1 and model == "8b") else None,
            "traffic_source": TRAFFIC_NCU["source"] if (world == 1 and model == "8b") else None,
            "peak_source": pk["src"], "algorithmic_bytes_per_launch": launch_bytes, "launch_ms": launch_ms,
            "launches_per_step": 1 if world == 1 else 2, "share_of_step": 1.0}
    if world > 1:
        roof["note"] = (f"rank 0 launches two kernels per token ({n_local}/{cfg.num_hidden_layers} layers, then the head after the ring "
                        "comes back); the second waits inside the kernel for the other shards, so this fraction is bytes of rank 0's "
                        "shard + head over the time of ALL shards — see token_roofline for the whole-token figure")
    if isolated:
        roof["isolated_per_op_kernels"] = isolated_kernels(sh, pk["hbm"])
    line = {
        "metric": metric_name(model), "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_all / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": (f"{MODEL_LABEL[model]} bf16, bs=1 decode, 2k context, layers sharded over {world} B200 (contiguous ranges, "
                                "one hidden-state hand-off per boundary)") if world > 1
                   else f"{MODEL_LABEL[model]} bf16, 1xB200, bs=1 decode, 2k context" + (" (BASELINE.json configs[1])" if model == "8b" else ""),
                   "kv_len_start": CTX_LEN + W, "kv_cache": "synthetic fill to 2048 positions (prefill is outside the metric, master.rs:131-134)",
                   "weights": "random-init N(0,0.02) bf16, HF layout, seed 1234", "greedy": True,
                   "parallelism": f"pp{world}" if world > 1 else "single",
                   "layers_per_rank": [len(r) for r in __import__("cake_b200.parallel", fromlist=["layer_split"]).layer_split(cfg.num_hidden_layers, world)],
                   "handoff": (os.environ.get("CAKE_B200_RING", "p2p") + (" (fused into the decode kernel over NVLink peer memory)" if os.environ.get("CAKE_B200_RING", "p2p") == "p2p" else " (ncclSend/ncclRecv graph nodes)")) if world > 1 else None,
                   "timing": "one enqueue of W+K graph replays, CUDA events after replay W and W+K on the library stream, max over ranks",
                   "l2": "inputs (GBs of weights per step) larger than L2; no flush needed"},
        "clocks": clocks,
        "gpu_launches": int(launches),
        "roofline": roof,
        "token_roofline": {"bytes_per_token": bpt, "achieved_GB_s": bpt / (ms_all / K * 1e-3) / 1e9,
                           "frac_of_one_gpu_hbm": bpt / (ms_all / K * 1e-3) / 1e9 / pk["hbm"],
                           "frac_of_aggregate_hbm": bpt / (ms_all / K * 1e-3) / 1e9 / (pk["hbm"] * world),
                           "roofline_tok_s_single_stream": pk["hbm"] * 1e9 / bpt,
                           "note": "bs=1 over a layer pipeline keeps one GPU busy at a time: the single-stream ceiling does not grow with N"},
    }
    if lat:
        lat_ms = sorted(x * 1e3 for x in lat)
        line["e2e"] = {"value": n_e2e / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4, "steps": n_e2e,
                       "warmup": E2E_WARM, "ms_per_step_p50": lat_ms[len(lat_ms) // 2], "ms_per_step_p99": lat_ms[min(len(lat_ms) - 1, int(len(lat_ms) * 0.99))],
                       "ms_per_step_max": lat_ms[-1],
                       "api": "cake_b200_decode_step_host (token id from host, sampled token back to host, sync per token)"}
    st = step_stats(traces, K, ms_all)
    if st:
        line["steps_trace"] = st
    if all_tokens:
        line["tokens_sha"] = hashlib.sha256(",".join(map(str, all_tokens)).encode()).hexdigest()[:16]
        line["tokens_head"] = all_tokens[:8]
    if par is not None:
        cpu = par.pop("cpu_baseline", None)
        line["parity"] = par
        if cpu:
            line["cpu_baseline"] = cpu
    sh.close()
    return line


TRAFFIC_NCU = {"bytes": 15280381000 + 8281856,
               "source": "dram__bytes_read.sum + dram__bytes_write.sum of one decode_mega_kernel launch, ncu --set full at N=1 "
                         "(profiles/mega_r02_raw.csv); cited from the committed capture, not measured in this run"}


def step_stats(traces, K: int, ms_all: float):
    """Per-rank split of a step into waiting for the input (inbox) and running, from the kernels' own %globaltimer
    stamps; the hop cost is what is left of a step after every shard's busy time."""
    try:
        per_rank = []
        step_busy = [0.0] * K
        for r, tr in enumerate(traces):
            if not tr:
                return None
            wait, busy = [], []
            for i, s in enumerate(tr):
                w = b = 0.0
                for o in (0, 4):
                    if s[o] and s[o + 2]:
                        w += (s[o + 1] - s[o]) / 1e3
                        b += (s[o + 2] - s[o + 1]) / 1e3
                wait.append(w)
                busy.append(b)
                step_busy[i] += b
            per_rank.append({"rank": r, "busy_us_p50": round(statistics.median(busy), 1), "busy_us_max": round(max(busy), 1),
                             "wait_us_p50": round(statistics.median(wait), 1)})
        # rank 0's own stamps bound each step: entry of the layers kernel of step i -> exit of its last kernel
        t0 = traces[0]
        dur = []
        for s in t0:
            end = s[6] if s[6] else s[2]
            dur.append((end - s[0]) / 1e3)
        hops = len(traces) if len(traces) > 1 else 0
        out = {"per_rank": per_rank, "step_us_p50": round(statistics.median(dur), 1), "step_us_p99": round(sorted(dur)[min(K - 1, int(K * 0.99))], 1),
               "step_us_max": round(max(dur), 1), "slowest_step": int(max(range(K), key=lambda i: dur[i]))}
        if hops:
            rest = [d - b for d, b in zip(dur, step_busy)]
            out["handoff_us_per_hop_p50"] = round(statistics.median(rest) / hops, 2)
            out["hops_per_step"] = hops
        return out
    except Exception as e:  # noqa: BLE001
        return {"error": str(e)}


def isolated_kernels(sh: Shard, peak: float) -> dict:
    """The same GEMV / attention phases timed live as stand-alone kernels (cake_b200_bench_kernel) — an aid that shows
    what each phase reaches without the phase boundaries, reported separately and never as the headline fraction."""
    import ctypes
    from cake_b200.capi import byref, check, int_array, lib, ptr_array
    cfg = sh.cfg
    H, I = cfg.hidden_size, cfg.intermediate_size
    try:
        hs, ix = ptr_array([b.h for b in sh.blocks]), int_array(sh.idx)
        per_kernel = {}
        kb = {0: 2 * (cfg.size_q + 2 * cfg.size_kv) * H, 1: 2 * H * cfg.size_q, 2: 2 * 2 * I * H, 3: 2 * H * I}
        names = {0: "qkv_gemv", 1: "o_gemv", 2: "gate_up_gemv", 3: "down_gemv", 4: "attn_decode"}
        for which in (2, 3, 0, 1, 4):
            msl = ctypes.c_float()
            check(lib().cake_b200_bench_kernel(sh.ctx.h, hs, ix, len(sh.blocks), sh.ctx.cache.h, which, 20, byref(msl)))
            nbytes = kb.get(which, 2 * 2 * cfg.num_key_value_heads * cfg.hd * sh.ctx.cache.len(sh.idx[0]))
            per_kernel[names[which]] = {"ms": round(msl.value, 5), "GB/s": round(nbytes / (msl.value * 1e-3) / 1e9, 1),
                                        "frac": round(nbytes / (msl.value * 1e-3) / 1e9 / peak, 4)}
        return {"what": "the same phases as stand-alone kernels (gemv_kernel / attn_decode_kernel), 20 launches each over distinct "
                        "layers, timed live; not part of the timed decode step", **per_kernel}
    except Exception as e:  # noqa: BLE001 - keep the headline line even if the aid fails
        return {"error": str(e)}


def parity_leg(env: Env, sh: Shard, all_tokens, cpu_leg: bool):
    """Restart from the same state as the timed run (KV refilled to CTX_LEN with the same pattern, first token 17) and
    check the first N_PARITY tokens against the oracle run on the host over the very same weights and cache:
    logits per step (bf16 ulps at the top binade), the in-kernel argmax, and the free-running greedy tokens of the
    timed run.  All ranks take part in the GPU steps; rank 0 owns the oracle."""
    import numpy as np
    import torch
    from cake_b200.capi import byref, c_uint32, check, lib
    from cake_b200.model import Cache
    cfg, rank = sh.cfg, env.rank
    oracle_feed, ref_logits, ref_toks, cpu = None, None, None, None
    sh.fill(CTX_LEN)
    if rank == 0:
        from oracle import oracle as O
        from tests.util import max_ulp_err, ulp_at_scale
        t_setup = time.perf_counter()
        for i in range(cfg.num_hidden_layers):     # host copies of the layers that live on other ranks (same seed -> same values)
            if f"{cfg.layer_name(i)}.input_layernorm.weight" not in sh.sd.host:
                sh.sd.get(f"{cfg.layer_name(i)}.input_layernorm.weight")
        sh.sd.drop_layers()
        torch.cuda.empty_cache()
        nthreads = oracle_threads()
        om = O.OracleModel(cfg, sh.sd.host, "bf16", max_seq=CTX_LEN + 64)
        oc = om.new_cache(CTX_LEN + 64)
        tmp = Cache(sh.ctx, 1, sh.cache_cap)       # the synthetic pattern depends on (seed, layer, capacity) only
        for l in range(cfg.num_hidden_layers):
            tmp.fill_synthetic([l], CTX_LEN, KV_SEED)
            k, v = tmp.kv(l)
            ko, vo = oc.kv(l)
            ko[:, :CTX_LEN] = k[0].float().numpy()
            vo[:, :CTX_LEN] = v[0].float().numpy()
            oc.set_len(l, CTX_LEN)
        tmp.close()
        setup_s = time.perf_counter() - t_setup
        # how far do two CORRECT implementations differ at this depth?  The reference pins "f32 accumulate", not the order
        # of the additions: re-run the first token with the oracle's two other summation orders (cake_oracle.c dot modes)
        alt = []
        for mode in (1, 2):
            O.set_dot_mode(mode)
            try:
                alt.append(om.forward([FIRST_TOKEN], CTX_LEN, oc))
            finally:
                O.set_dot_mode(0)
            for l in range(cfg.num_hidden_layers):
                oc.set_len(l, CTX_LEN)
        res = time_oracle_tokens(om, oc, FIRST_TOKEN, CTX_LEN, N_PARITY + (2 if cpu_leg else 0), 40.0)
        ref_toks, ref_logits = res["tokens"], res["logits"]
        sens = max(max_ulp_err(a_, ref_logits[0], "bf16") for a_ in alt)
        oracle_feed = [FIRST_TOKEN] + ref_toks[:N_PARITY - 1]
        if cpu_leg:
            t = res["times"][1:] if len(res["times"]) > 1 else res["times"]   # the first token pages the weights in
            cpu = {"value": 1.0 / statistics.mean(t), "unit": "tok/s", "cores": nthreads, "kind": "port",
                   "sample": f"{len(t)} decode tokens of the full {cfg.num_hidden_layers}-layer model at KV length {CTX_LEN}+ on the real weights "
                             f"(oracle/cake_oracle.c, OpenMP bound to the physical cores of one socket; 1 untimed warm-up token; setup {setup_s:.0f}s)",
                   "spread_tok_s": {"min": 1.0 / max(t), "median": 1.0 / statistics.median(t), "max": 1.0 / min(t)},
                   "host": host_info()}
    sh.begin(FIRST_TOKEN)
    env.barrier()
    steps = []
    if rank == 0:
        logits = torch.empty(cfg.vocab_size, dtype=torch.bfloat16)
        for i, tok_in in enumerate(oracle_feed):
            nxt = c_uint32()
            check(lib().cake_b200_decode_step_host(sh.ctx.h, tok_in, byref(nxt)))
            check(lib().cake_b200_decode_logits(sh.ctx.h, logits.data_ptr(), logits.numel() * 2))
            lg = logits.float().numpy()
            ref = ref_logits[i]
            srt = np.sort(ref)
            u = ulp_at_scale(ref, "bf16")
            steps.append({"token_in": int(tok_in), "gpu_token": int(nxt.value), "oracle_token": int(ref_toks[i]),
                          "max_logit_err_ulp": round(max_ulp_err(lg, ref, "bf16"), 3),
                          "oracle_margin_ulp": round(float(srt[-1] - srt[-2]) / u, 2),
                          "argmax_of_gpu_logits": int(O.argmax(lg))})
        sh.pos += len(oracle_feed)
    else:
        sh.run(N_PARITY)
        sh.wait(sh.event())
    env.barrier()
    if rank != 0:
        return None
    tol = max(4.0, 2.0 * sens)
    ok = all(s["max_logit_err_ulp"] <= tol and s["gpu_token"] == s["argmax_of_gpu_logits"] and
             (s["gpu_token"] == s["oracle_token"] or s["oracle_margin_ulp"] <= 2 * tol) for s in steps)
    free_run = all_tokens[:N_PARITY] if all_tokens else None
    return {"checked_against": "oracle/cake_oracle.c on the same weights and KV cache (host), teacher-forced on the oracle's tokens",
            "tolerance_ulp_bf16": round(tol, 2), "tolerance_rule": "max(4, 2 x order sensitivity) bf16 ulps at the logits' top binade",
            "oracle_order_sensitivity_ulp": round(sens, 2),
            "oracle_order_sensitivity_what": "max logit difference between the oracle and itself with a second f32 summation order / f64 "
                                             "accumulation in its linear layers (same token): what 32 layers of bf16 roundings do to two correct implementations",
            "steps": steps, "ok": bool(ok),
            "timed_run_first_tokens": free_run, "oracle_first_tokens": [int(t) for t in ref_toks[:N_PARITY]],
            "timed_run_matches_oracle": (free_run == [int(t) for t in ref_toks[:N_PARITY]]) if free_run else None,
            "cpu_baseline": cpu}


# ------------------------------------------------------------------------------------------------
def config0_leg(env: Env) -> dict:
    """BASELINE configs[0]: Qwen3-0.6B (28 layers, f16 = the reference's default dtype), greedy decode of 32 tokens from
    one 16-token prompt: the GPU through Master.generate_text (tok/s by the reference's definition, master.rs:131-166)
    and through the decode graph, next to the oracle port on the host cores; tokens compared."""
    import numpy as np
    import torch
    from cake_b200.config import qwen3_0_6b
    from cake_b200.model import Context, Master, TextModelBase
    from cake_b200.synth import LazyCheckpoint
    from oracle import oracle as O
    from tests.util import max_ulp_err, ulp_at_scale
    cfg = qwen3_0_6b(max_seq=256)
    sd = LazyCheckpoint(cfg, "f16", seed=2024, device=env.dev, std=0.03, host_copy=True)
    ctx = Context(cfg, sd, "f16", device=env.local, max_seq=256)
    model = TextModelBase.load(ctx)
    sd.drop_layers()
    prompt = np.random.default_rng(1).integers(0, cfg.vocab_size, 16).tolist()
    n_new = 32
    Master(model).generate_text(prompt, 4)                      # warm-up
    out = Master(model).generate_text(prompt, n_new)            # host-stepped: prefill + 31 decode steps through next_token
    # graph path: prefill through next_token(0), then 31 greedy tokens fed back on the device
    model.prepare_prompt(prompt)
    t0 = model.next_token(0).id
    model.decode_build()
    model.decode_greedy(t0, 4)
    model.prepare_prompt(prompt)
    t0 = model.next_token(0).id
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx.sync()
    e0.record(ctx.torch_stream)
    g = model.decode_greedy(t0, n_new - 1)
    e1.record(ctx.torch_stream)
    ctx.sync()
    graph_tok_s = (n_new - 1) / (e0.elapsed_time(e1) / 1e3)
    nthreads = oracle_threads()
    om = O.OracleModel(cfg, sd.host, "f16", max_seq=256)
    oc = om.new_cache(256)
    om.generate(prompt, 2, oc)
    t1 = time.perf_counter()
    ref_toks, ref_logits = om.generate(prompt, n_new, oc)
    cpu_s = time.perf_counter() - t1
    # teacher-forced logits check over the 32 steps
    model.prepare_prompt(prompt)
    feeds = [prompt] + [[t] for t in ref_toks[:-1]]
    pos, worst, flips, out_margin = 0, 0.0, 0, 0
    for step, ids in enumerate(feeds):
        lg = model.forward([ids], pos)
        ctx.sync()
        lg = lg[0].float().cpu().numpy()
        pos += len(ids)
        worst = max(worst, max_ulp_err(lg, ref_logits[step], "f16"))
        if O.argmax(lg) != ref_toks[step]:
            flips += 1
            srt = np.sort(ref_logits[step])
            if float(srt[-1] - srt[-2]) > 2 * 4.0 * ulp_at_scale(ref_logits[step], "f16"):
                out_margin += 1
    nmatch = 0
    for a, b in zip(out["tokens"], ref_toks):
        if a != b:
            break
        nmatch += 1
    wb = 2.0 * (cfg.num_hidden_layers * (cfg.hidden_size * (cfg.size_q + 2 * cfg.size_kv) + cfg.size_q * cfg.hidden_size + 3 * cfg.hidden_size * cfg.intermediate_size)
                + cfg.vocab_size * cfg.hidden_size)
    res = {"workload": "Qwen3-0.6B (28 layers, QK-norm, tied head), f16, 16-token prompt, greedy 32 tokens (BASELINE.json configs[0])",
           "gpu_tok_s_generate_text": out["tok_s"], "gpu_tok_s_decode_graph": graph_tok_s,
           "gpu_hbm_frac_decode_graph": wb * graph_tok_s / 1e9 / peaks()["hbm"],
           "cpu_baseline": {"value": n_new / cpu_s, "unit": "tok/s", "cores": nthreads, "kind": "port",
                            "sample": "the same 32 tokens (prefill of 16 included) through the oracle port, 28 layers"},
           "tokens_equal_prefix": nmatch, "tokens_total": n_new, "graph_tokens_equal_generate_text": ([t0] + g) == out["tokens"],
           "teacher_forced": {"worst_logit_err_ulp_f16": round(worst, 3), "argmax_flips": flips, "flips_outside_margin": out_margin},
           "ok": bool(out_margin == 0 and worst <= 8.0)}
    ctx.close()
    torch.cuda.empty_cache()
    return res


def prefill_leg(env: Env, reps: int = 3, batch: int = 32, seq: int = 4096) -> dict:
    """BASELINE configs[4]: Llama-3-8B bf16, bs=32 x 4096 prefill on one B200 — one Forwarder::forward_batch over all
    32 blocks from an empty cache (x: (32, 4096, 4096)) + ln_f / lm_head on the last position of each row
    (text_model.rs:336-352).  Tensor-bound: algorithmic FLOPs over the measured time against the
    measured sustained bf16 tensor throughput."""
    import torch
    from cake_b200.capi import check, lib, ptr
    from cake_b200.model import Cache, Context, TextModelBase
    from cake_b200.synth import LazyCheckpoint
    cfg = model_config("8b", seq)
    sd = LazyCheckpoint(cfg, "bf16", seed=1234, device=env.dev)
    ctx = Context(cfg, sd, "bf16", device=env.local, max_seq=seq)
    ctx.cache = Cache(ctx, batch, seq)
    model = TextModelBase.load(ctx)
    sd.drop_layers()
    sd.drop_head()
    torch.cuda.empty_cache()
    blks = model.blocks
    nl = len(blks)
    with torch.cuda.stream(ctx.torch_stream):
        g = torch.Generator(device=env.dev).manual_seed(11)
        x = (torch.randn(batch, seq, cfg.hidden_size, generator=g, device=env.dev) * 0.5).to(torch.bfloat16)
        logits = torch.empty(batch, cfg.vocab_size, dtype=torch.bfloat16, device=env.dev)
    bl = [(b.layer_name(), 0, i) for i, b in enumerate(blks)]
    times = []
    l0 = 0
    for rep in range(reps + 1):
        ctx.cache.clear()
        ctx.sync()
        if rep == reps and env.sampler:
            env.sampler.start()
        l0 = ctx.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ctx.torch_stream)
        y = blks[0].forward_batch(x, bl, ctx, blocks=blks)
        check(lib().cake_b200_logits(ctx.h, ptr(y), batch, seq, ptr(logits), None))
        e1.record(ctx.torch_stream)
        ctx.sync()
        if rep > 0:
            times.append(e0.elapsed_time(e1))
    clocks = env.sampler.stop() if env.sampler else None
    launches = ctx.launch_count() - l0
    finite = bool(torch.isfinite(logits.float()).all())
    H, I = cfg.hidden_size, cfg.intermediate_size
    M = batch * seq
    flop_lin = 2.0 * M * (cfg.size_q + 2 * cfg.size_kv + cfg.size_q + 3 * I) * H * nl
    flop_att = 2.0 * 2 * batch * cfg.num_attention_heads * cfg.hd * seq * seq / 2 * nl
    flop_head = 2.0 * batch * cfg.vocab_size * H
    flops = flop_lin + flop_att + flop_head
    ms = statistics.median(times)
    pk = peaks()
    res = {"metric": "prefill tok/s (Llama-3-8B bf16, bs=32 x 4096)", "value": M / (ms / 1e3), "unit": "tok/s", "ms_per_step": ms,
           "steps": reps, "warmup": 1, "finite": finite,
           "config": {"workload": "Llama-3-8B bf16, 1xB200, bs=32 prefill at 4k seq, all 32 layers + last-position lm_head (BASELINE.json configs[4])",
                      "l2": "activations of one step (1 GB per (32,4096,4096) tensor) larger than L2; no flush needed"},
           "gpu_launches": int(launches), "clocks": clocks,
           "roofline": {"bound": "tensor", "achieved": round(flops / (ms * 1e-3) / 1e12, 1), "peak": pk["tc"], "unit": "TFLOP/s",
                        "frac": round(flops / (ms * 1e-3) / 1e12 / pk["tc"], 4), "traffic": None,
                        "peak_source": pk["src"] + " (sustained cuBLAS bf16, the kernel runs inside a seconds-long step)",
                        "algorithmic_flops_per_step": flops,
                        "flops_split": {"linears": flop_lin, "causal_attention": flop_att, "lm_head": flop_head},
                        "kernels": "per layer: gemm_tc_kernel (tcgen05, 128x256 tiles, TMA-multicast CTA pairs) x4 + attn_prefill_tc_kernel (tcgen05 flash attention) + rmsnorm_rows_vec x2 + rope_append_vec; ncu: profiles/launches_prefill_r02.csv"}}
    ctx.close()
    torch.cuda.empty_cache()
    return res



# ------------------------------------------------------------------------------------------------
NIGENEX_SIZES = {  # layer sizes of real models, 4 layers each (random weights): width, heads, kv_heads, head_dim, ff, window
    "2k": dict(width=2048, heads=16, kv_heads=4, head_dim=128, ff=8192, window=1024),
    "4k": dict(width=4096, heads=32, kv_heads=8, head_dim=128, ff=14336, window=1024),
    "4k-hd64": dict(width=4096, heads=64, kv_heads=8, head_dim=64, ff=14336, window=1024),
}


def nigenex_leg(env: Env, sizes=("2k", "4k", "4k-hd64"), n_layers: int = 4, batch: int = 4, seq: int = 4096, ctx_len: int = 2048,
                steps: int = 32, reps: int = 3) -> dict:
    """`--workload nigenex`: the Nigenex design (layer-list blocks, fp32 residual stream) beside the framework's closest
    existing model at equal layer sizes — the Gemma3-style block (per-layer sliding window without RoPE, tanh-gelu MLP,
    stepped through the same batched path) — both through TextModelBase / forward_batch:
      prefill   one step of batch x seq tokens from an empty cache through all layers + the head on the last positions
      decode    bs=1: a ctx_len-token prompt, then `steps` single-token steps (embed -> layers -> head), timed as a whole
    Device time by CUDA events on the library's stream.  L2: the step's activations (prefill) / the layers' weights (decode)
    exceed the 126 MB L2 at every size."""
    import torch
    from cake_b200.capi import check, lib, ptr
    from cake_b200.config import Config, LayerSpec
    from cake_b200.model import Cache, Context, TextModelBase
    from cake_b200.synth import make_checkpoint, make_listed_checkpoint
    pk = peaks()
    out = {}
    launches = 0
    for name in sizes:
        z = NIGENEX_SIZES[name]
        W, nh, nkv, hd, ff, win = z["width"], z["heads"], z["kv_heads"], z["head_dim"], z["ff"], z["window"]
        vocab = 32768
        row = {"size": z}
        for arch in ("nigenex", "closest"):
            if arch == "nigenex":
                spec = LayerSpec(heads=nh, kv_heads=nkv, head_dim=hd, window=win, scale=hd ** -0.5, softcap=30.0, ff=ff)
                cfg = Config(hidden_size=W, intermediate_size=ff, vocab_size=vocab, num_hidden_layers=n_layers, num_attention_heads=nh,
                             num_key_value_heads=nkv, head_dim=hd, max_seq_len=seq, block_kind="nigenex", layers=[spec] * n_layers,
                             logit_softcap=30.0, model_prefix="")
                sd = make_listed_checkpoint(cfg, "bf16", seed=5, device=env.dev, std=0.02)
                n_in = (nh + nkv) * hd + nh
                flop_lin = 2.0 * W * (n_in + 2 * ff + nh * hd + ff)
                wbytes = 2.0 * W * (n_in + 3 * ff + nh * hd)
                att_keys = lambda S: sum(min(i + 1, win) for i in range(S))
            else:
                cfg = Config(hidden_size=W, intermediate_size=ff, vocab_size=vocab, num_hidden_layers=n_layers, num_attention_heads=nh,
                             num_key_value_heads=nkv, head_dim=hd, max_seq_len=seq, block_kind="gemma3", sliding_window=win,
                             global_layers=[False] * n_layers, use_qk_norm=True, use_gelu_mlp=True, tie_word_embeddings=True)
                sd = make_checkpoint(cfg, "bf16", seed=5, device=env.dev, std=0.02)
                flop_lin = 2.0 * W * ((nh + 2 * nkv) * hd + 2 * ff + nh * hd + ff)
                wbytes = 2.0 * W * ((nh + 2 * nkv) * hd + 3 * ff + nh * hd)
                att_keys = lambda S: S * (S + 1) // 2   # the first call on an empty cache attends over everything it stores (cache.rs:173-205)
            ctx = Context(cfg, sd, "bf16", device=env.local, max_seq=seq)
            model = TextModelBase.load(ctx)
            del sd
            torch.cuda.empty_cache()
            blks = model.blocks
            bl = [(b.layer_name(), 0, i) for i, b in enumerate(blks)]
            # ---- prefill
            ctx.cache = Cache(ctx, batch, seq)
            with torch.cuda.stream(ctx.torch_stream):
                g = torch.Generator(device=env.dev).manual_seed(11)
                x = (torch.randn(batch, seq, W, generator=g, device=env.dev) * 0.5).to(ctx.stream_dtype)
                logits = torch.empty(batch, vocab, dtype=ctx.logits_dtype, device=env.dev)
            times = []
            for r in range(reps + 1):
                ctx.cache.clear()
                ctx.sync()
                l0 = ctx.launch_count()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(ctx.torch_stream)
                y = blks[0].forward_batch(x, bl, ctx, blocks=blks)
                check(lib().cake_b200_logits(ctx.h, ptr(y), batch, seq, ptr(logits), None))
                e1.record(ctx.torch_stream)
                ctx.sync()
                if r > 0:
                    times.append(e0.elapsed_time(e1))
                    launches += ctx.launch_count() - l0
            ms = statistics.median(times)
            M = batch * seq
            flops = n_layers * (flop_lin * M + 4.0 * nh * hd * batch * att_keys(seq)) + 2.0 * batch * vocab * W
            pre = {"tok_s": M / (ms / 1e3), "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
                   "frac_of_tensor_peak": flops / (ms * 1e-3) / 1e12 / pk["tc"], "finite": bool(torch.isfinite(logits.float()).all())}
            del x, y
            # ---- decode
            ctx.cache = Cache(ctx, 1, seq)
            ids = torch.randint(0, vocab, (ctx_len + steps + 3,), generator=torch.Generator().manual_seed(3)).tolist()
            model.forward([ids[:ctx_len]], 0)
            pos = ctx_len
            for _ in range(3):
                model.forward([[ids[pos]]], pos)
                pos += 1
            ctx.sync()
            l0 = ctx.launch_count()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(ctx.torch_stream)
            for _ in range(steps):
                lg = model.forward([[ids[pos]]], pos)
                pos += 1
            e1.record(ctx.torch_stream)
            ctx.sync()
            launches += ctx.launch_count() - l0
            dms = e0.elapsed_time(e1) / steps
            dbytes = n_layers * (wbytes + 2.0 * nkv * hd * min(win, ctx_len) * (1 if arch == "nigenex" else 2)) + 2.0 * vocab * W
            dec = {"tok_s": 1e3 / dms, "ms_per_token": dms, "gb_s": dbytes / (dms * 1e-3) / 1e9, "frac_of_hbm_peak": dbytes / (dms * 1e-3) / 1e9 / pk["hbm"],
                   "finite": bool(torch.isfinite(lg.float()).all())}
            row[arch] = {"prefill": pre, "decode": dec}
            ctx.close()
            del model, blks, ctx
            torch.cuda.empty_cache()
        row["prefill_ratio"] = row["nigenex"]["prefill"]["tok_s"] / row["closest"]["prefill"]["tok_s"]
        row["decode_ratio"] = row["nigenex"]["decode"]["tok_s"] / row["closest"]["decode"]["tok_s"]
        out[name] = row
    head = out[sizes[-1] if "4k" not in out else "4k"]
    return {"metric": "nigenex prefill tok/s (4 layers of Llama-3-8B size, bf16, bs=4 x 4096)", "value": head["nigenex"]["prefill"]["tok_s"],
            "unit": "tok/s", "ms_per_step": head["nigenex"]["prefill"]["ms"], "steps": reps, "warmup": 1, "gpu_launches": int(launches),
            "config": {"workload": f"Nigenex vs the Gemma3-style windowed block at equal sizes, {n_layers} layers, bf16, prefill bs={batch} x {seq}, "
                                   f"decode bs=1 at {ctx_len} context x {steps} steps", "l2": "prefill activations / decode weights exceed L2"},
            "peaks": {"tensor_tflops": pk["tc"], "hbm_gbs": pk["hbm"], "source": pk["src"]}, "sizes": out}

SETODRA_SIZES = {  # layer sizes of real models (random weights): retention / state-space / state-space / latent attention, each with a routed feed-forward
    "1k": dict(width=1024, ret=dict(heads=8, dim=128, vdim=128), ssd=dict(heads=32, vdim=64, state=128, groups=4, conv=4, norm_groups=4),
               lat=dict(heads=8, dim=128, rot_dim=64, vdim=128, kv_rank=512), moe=dict(experts=32, identity=2, top=4, ff=704, shared_ff=1408)),
    "2k": dict(width=2048, ret=dict(heads=16, dim=128, vdim=128), ssd=dict(heads=64, vdim=64, state=128, groups=8, conv=4, norm_groups=8),
               lat=dict(heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512), moe=dict(experts=64, identity=2, top=6, ff=1408, shared_ff=2816)),
}


def setodra_leg(env: Env, sizes=("1k", "2k"), batch: int = 4, seq: int = 4096, ctx_len: int = 2048, steps: int = 32, reps: int = 3) -> dict:
    """`--workload setodra`: the Setodra design (mixer-list blocks: retention, two state-space layers, latent attention, each
    followed by a routed feed-forward) beside the framework's closest existing model, Nigenex (the other layer-list model
    with an fp32 residual stream), at equal width, layer count and active feed-forward width per token, both through
    TextModelBase / forward_batch:
      prefill   one step of batch x seq tokens from an empty cache through all layers + the head on the last positions
      decode    bs=1: a ctx_len-token prompt, then `steps` single-token steps (embed -> layers -> head), timed as a whole
    Device time by CUDA events on the library's stream; activations (prefill) / weights (decode) exceed the 126 MB L2."""
    import torch
    from cake_b200.capi import check, lib, ptr
    from cake_b200.config import Config, LayerSpec, MixerSpec, MoeSpec, RotarySpec
    from cake_b200.model import Cache, Context, TextModelBase
    from cake_b200.synth import make_listed_checkpoint, make_mixer_checkpoint
    pk = peaks()
    out, launches, vocab = {}, 0, 32768
    mseq = max(seq, ctx_len + steps + 8)
    for name in sizes:
        z = SETODRA_SIZES[name]
        W, mo = z["width"], MoeSpec(scale=2.5, **z["moe"])
        row = {"size": z}
        for arch in ("setodra", "closest"):
            if arch == "setodra":
                rot = RotarySpec(dims=z["lat"]["rot_dim"], base=10000.0, factor=8.0, fast=32.0, slow=1.0, original=2048)
                layers = [MixerSpec(type="retention", decay=[1 - 2.0 ** (-5 - i % 4) for i in range(z["ret"]["heads"])],
                                    rot=RotarySpec(dims=z["ret"]["dim"], base=10000.0), moe=mo, **z["ret"]),
                          MixerSpec(type="mamba2", moe=mo, **z["ssd"]), MixerSpec(type="mamba2", moe=mo, **z["ssd"]),
                          MixerSpec(type="latent_attention", scale=(z["lat"]["dim"] + z["lat"]["rot_dim"]) ** -0.5, rot=rot, moe=mo, **z["lat"])]
                cfg = Config(hidden_size=W, intermediate_size=0, vocab_size=vocab, num_hidden_layers=len(layers), num_attention_heads=layers[0].heads,
                             num_key_value_heads=layers[0].heads, rms_norm_eps=1e-6, head_dim=128, max_seq_len=mseq, block_kind="setodra",
                             layers=layers, model_prefix="", embed_scale=1.0)
                sd = make_mixer_checkpoint(cfg, "bf16", seed=5, device=env.dev, std=0.02)
                r, m2, la = z["ret"], z["ssd"], z["lat"]
                n_in = [2 * r["heads"] * r["dim"] + 2 * r["heads"] * r["vdim"], 2 * m2["heads"] * m2["vdim"] + 2 * m2["groups"] * m2["state"] + m2["heads"],
                        la["heads"] * (la["dim"] + la["rot_dim"]) + la["kv_rank"] + la["rot_dim"]]
                inner = [r["heads"] * r["vdim"], m2["heads"] * m2["vdim"], la["heads"] * la["vdim"]]
                ff_act = mo.top * mo.ff + mo.shared_ff
                lin = [2.0 * W * (n_in[i] + inner[i]) for i in (0, 1, 1, 2)]
                lat_up = 2.0 * la["heads"] * la["kv_rank"] * (la["dim"] + la["vdim"])
                flop_tok = sum(lin) + lat_up + 4 * (2.0 * W * 3 * ff_act + 2.0 * W * (mo.experts + mo.identity))
                flop_tok += 4.0 * r["heads"] * r["dim"] * r["vdim"] + 2 * 4.0 * m2["heads"] * m2["state"] * m2["vdim"]   # state update + read-out
                att_flops = lambda S: 2.0 * la["heads"] * (2 * la["kv_rank"] + la["rot_dim"]) * (S * (S + 1) // 2)
                wbytes = sum(lin) + lat_up + 4 * (2.0 * W * 3 * ff_act)     # 2 bytes per weight read once = its FLOPs per token
                state_bytes = 8.0 * (r["heads"] * r["dim"] * r["vdim"] + 2 * m2["heads"] * m2["state"] * m2["vdim"]) + 2.0 * ctx_len * (la["kv_rank"] + la["rot_dim"])
            else:
                nh = W // 128
                ffn = mo.top * mo.ff + mo.shared_ff
                spec = LayerSpec(heads=nh, kv_heads=max(1, nh // 4), head_dim=128, window=1024, scale=128 ** -0.5, softcap=30.0, ff=ffn)
                cfg = Config(hidden_size=W, intermediate_size=ffn, vocab_size=vocab, num_hidden_layers=4, num_attention_heads=nh,
                             num_key_value_heads=spec.kv_heads, head_dim=128, max_seq_len=mseq, block_kind="nigenex", layers=[spec] * 4,
                             logit_softcap=30.0, model_prefix="")
                sd = make_listed_checkpoint(cfg, "bf16", seed=5, device=env.dev, std=0.02)
                n_in1 = (nh + spec.kv_heads) * 128 + nh
                flop_tok = 4 * 2.0 * W * (n_in1 + 3 * ffn + nh * 128)
                att_flops = lambda S: 4 * 4.0 * nh * 128 * sum(min(i + 1, 1024) for i in range(S))
                wbytes = flop_tok
                state_bytes = 4 * 2.0 * spec.kv_heads * 128 * min(1024, ctx_len)
            ctx = Context(cfg, sd, "bf16", device=env.local, max_seq=mseq)
            model = TextModelBase.load(ctx)
            del sd
            torch.cuda.empty_cache()
            # ---- prefill
            ctx.cache = Cache(ctx, batch, seq)
            ids = torch.randint(0, vocab, (batch, seq), generator=torch.Generator().manual_seed(11)).numpy()
            times = []
            for rr in range(reps + 1):
                ctx.cache.clear()
                ctx.sync()
                l0 = ctx.launch_count()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(ctx.torch_stream)
                logits = model.forward(ids, 0)
                e1.record(ctx.torch_stream)
                ctx.sync()
                if rr > 0:
                    times.append(e0.elapsed_time(e1))
                    launches += ctx.launch_count() - l0
            ms = statistics.median(times)
            M = batch * seq
            flops = flop_tok * M + batch * att_flops(seq) + 2.0 * batch * vocab * W
            pre = {"tok_s": M / (ms / 1e3), "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
                   "frac_of_tensor_peak": flops / (ms * 1e-3) / 1e12 / pk["tc"], "finite": bool(torch.isfinite(logits.float()).all())}
            # ---- decode
            ctx.cache = Cache(ctx, 1, mseq)
            ids1 = torch.randint(0, vocab, (ctx_len + steps + 3,), generator=torch.Generator().manual_seed(3)).tolist()
            model.forward([ids1[:ctx_len]], 0)
            pos = ctx_len
            for _ in range(3):
                model.forward([[ids1[pos]]], pos)
                pos += 1
            ctx.sync()
            l0 = ctx.launch_count()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(ctx.torch_stream)
            for _ in range(steps):
                lg = model.forward([[ids1[pos]]], pos)
                pos += 1
            e1.record(ctx.torch_stream)
            ctx.sync()
            launches += ctx.launch_count() - l0
            dms = e0.elapsed_time(e1) / steps
            dbytes = wbytes + state_bytes + 2.0 * vocab * W
            dec = {"tok_s": 1e3 / dms, "ms_per_token": dms, "gb_s": dbytes / (dms * 1e-3) / 1e9, "frac_of_hbm_peak": dbytes / (dms * 1e-3) / 1e9 / pk["hbm"],
                   "launches_per_token": (ctx.launch_count() - l0) / steps, "finite": bool(torch.isfinite(lg.float()).all())}
            row[arch] = {"prefill": pre, "decode": dec}
            ctx.close()
            del model, ctx
            torch.cuda.empty_cache()
        row["prefill_ratio"] = row["setodra"]["prefill"]["tok_s"] / row["closest"]["prefill"]["tok_s"]
        row["decode_ratio"] = row["setodra"]["decode"]["tok_s"] / row["closest"]["decode"]["tok_s"]
        out[name] = row
    head = out[sizes[-1]]
    return {"metric": f"setodra prefill tok/s (4 layers, width {head['size']['width']}, bf16, bs={batch} x {seq})", "value": head["setodra"]["prefill"]["tok_s"],
            "unit": "tok/s", "ms_per_step": head["setodra"]["prefill"]["ms"], "steps": reps, "warmup": 1, "gpu_launches": int(launches),
            "config": {"workload": f"Setodra vs Nigenex at equal width, layer count and active feed-forward width, 4 layers, bf16, prefill bs={batch} x {seq}, "
                                   f"decode bs=1 at {ctx_len} context x {steps} steps", "l2": "prefill activations / decode weights exceed L2"},
            "peaks": {"tensor_tflops": pk["tc"], "hbm_gbs": pk["hbm"], "source": pk["src"]}, "sizes": out}


NUVARAX_SIZES = {  # layer sizes of real models (random weights): [attention beside a matrix memory, delta rule] x 2, each with a dense feed-forward
    "1k": dict(width=1024, ff=4224, left=dict(heads=8, kv_heads=2, dim=128, vdim=128), right=dict(heads=4, dim=128, vdim=128),
               delta=dict(heads=8, kv_heads=8, dim=128, vdim=128, conv=4)),
    "2k": dict(width=2048, ff=11264, left=dict(heads=16, kv_heads=4, dim=128, vdim=128), right=dict(heads=8, dim=128, vdim=128),
               delta=dict(heads=16, kv_heads=16, dim=128, vdim=128, conv=4)),
}


def _time_listed_model(env: Env, cfg, sd, batch: int, seq: int, ctx_len: int, steps: int, reps: int, mseq: int) -> dict:
    """Prefill (one step of batch x seq tokens from an empty cache + the head on the last positions) and bs=1 decode (a
    ctx_len-token prompt, then `steps` single-token steps) of a layer-list model through TextModelBase; device time by CUDA events."""
    import torch
    from cake_b200.model import Cache, Context, TextModelBase
    vocab = cfg.vocab_size
    ctx = Context(cfg, sd, "bf16", device=env.local, max_seq=mseq)
    model = TextModelBase.load(ctx)
    torch.cuda.empty_cache()
    ctx.cache = Cache(ctx, batch, seq)
    ids = torch.randint(0, vocab, (batch, seq), generator=torch.Generator().manual_seed(11)).numpy()
    times, launches = [], 0
    for rr in range(reps + 1):
        ctx.cache.clear()
        ctx.sync()
        l0 = ctx.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ctx.torch_stream)
        logits = model.forward(ids, 0)
        e1.record(ctx.torch_stream)
        ctx.sync()
        if rr > 0:
            times.append(e0.elapsed_time(e1))
            launches += ctx.launch_count() - l0
    pre = {"ms": statistics.median(times), "finite": bool(torch.isfinite(logits.float()).all()), "launches": (ctx.launch_count() - l0)}
    ctx.cache = Cache(ctx, 1, mseq)
    ids1 = torch.randint(0, vocab, (ctx_len + steps + 3,), generator=torch.Generator().manual_seed(3)).tolist()
    model.forward([ids1[:ctx_len]], 0)
    pos = ctx_len
    for _ in range(3):
        model.forward([[ids1[pos]]], pos)
        pos += 1
    ctx.sync()
    l0 = ctx.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ctx.torch_stream)
    for _ in range(steps):
        lg = model.forward([[ids1[pos]]], pos)
        pos += 1
    e1.record(ctx.torch_stream)
    ctx.sync()
    launches += ctx.launch_count() - l0
    dec = {"ms_per_token": e0.elapsed_time(e1) / steps, "launches_per_token": (ctx.launch_count() - l0) / steps, "finite": bool(torch.isfinite(lg.float()).all())}
    ctx.close()
    del model, ctx
    torch.cuda.empty_cache()
    return {"prefill": pre, "decode": dec, "launches": launches}


def nuvarax_leg(env: Env, sizes=("1k", "2k"), batch: int = 4, seq: int = 4096, ctx_len: int = 2048, steps: int = 32, reps: int = 3) -> dict:
    """`--workload nuvarax`: the Nuvarax design (mixer-list blocks with norms on both sides of every sublayer and an input
    convolution: attention with mixed heads beside a matrix memory, delta rule, attention + memory, delta rule, each followed by a
    dense clamped feed-forward) beside the framework's closest existing model, Setodra (the other mixer-list model: latent
    attention, retention, latent attention, retention, each with a routed feed-forward of the same active width), at equal width
    and layer count, both through TextModelBase / forward_batch.  Workload and timing as in the Setodra leg."""
    import torch
    from cake_b200.config import Config, MixerSpec, MoeSpec, RotarySpec
    from cake_b200.synth import make_mixer_checkpoint, make_nuvarax_checkpoint
    pk = peaks()
    out, launches, vocab = {}, 0, 32768
    mseq = max(seq, ctx_len + steps + 8)
    for name in sizes:
        z, zs = NUVARAX_SIZES[name], SETODRA_SIZES[name]
        W, ff = z["width"], z["ff"]
        row = {"size": z}
        for arch in ("nuvarax", "closest"):
            if arch == "nuvarax":
                a, b, dl = z["left"], z["right"], z["delta"]
                layer = lambda kind, m: {"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff, "limit": 7.0}}
                par = {"left": dict(scale=a["dim"] ** -0.5, bias_max=1024, **a), "right": dict(gate_cap=15.0, **b)}
                d = {"architecture": "Nuvarax", "width": W, "vocab": vocab, "norm": {"eps": 1e-6}, "max_positions": mseq, "canon": {"taps": 4},
                     "embedding": {"scale": 1.0, "bigram": {"buckets": 99991, "mul_prev": 1009, "mul_cur": 31}},
                     "layers": [layer("parallel", par), layer("delta", dl), layer("parallel", par), layer("delta", dl)]}
                cfg = Config.from_hf(d)
                cfg.max_seq_len = mseq
                sd = make_nuvarax_checkpoint(cfg, "bf16", seed=5, device=env.dev, std=0.02)
                Ha, Ga, Hb, Hd = a["heads"], a["kv_heads"], b["heads"], dl["heads"]
                n_par = Ha * a["dim"] + Ga * (a["dim"] + a["vdim"]) + Ha * a["vdim"] + 2 * Hb * b["dim"] + 2 * Hb * b["vdim"] + 2 * Hb
                n_del = 2 * dl["kv_heads"] * dl["dim"] + 2 * Hd * dl["vdim"] + 2 * Hd
                lin = 2 * 2.0 * W * (n_par + Ha * a["vdim"] + Hb * b["vdim"]) + 2 * 2.0 * W * (n_del + Hd * dl["vdim"])
                flop_tok = lin + 4 * 2.0 * W * 3 * ff
                flop_tok += 2 * 4.0 * Hb * b["dim"] * b["vdim"] + 2 * 6.0 * Hd * dl["dim"] * dl["vdim"]      # state updates + read-outs
                att_flops = lambda S: 2 * 2.0 * Ha * (a["dim"] + a["vdim"]) * (S * (S + 1) // 2)
                wbytes = flop_tok - (2 * 4.0 * Hb * b["dim"] * b["vdim"] + 2 * 6.0 * Hd * dl["dim"] * dl["vdim"])
                state_bytes = 2 * 8.0 * (Hb * b["dim"] * b["vdim"] + Hd * dl["dim"] * dl["vdim"]) + 2 * 2.0 * ctx_len * Ga * (a["dim"] + a["vdim"])
            else:
                mo = MoeSpec(scale=2.5, **zs["moe"])
                scale_ff = ff / float(mo.top * mo.ff + mo.shared_ff)   # the routed feed-forward at the dense one's active width
                mo.ff, mo.shared_ff = int(mo.ff * scale_ff) // 64 * 64, int(mo.shared_ff * scale_ff) // 64 * 64
                rot = RotarySpec(dims=zs["lat"]["rot_dim"], base=10000.0, factor=8.0, fast=32.0, slow=1.0, original=2048)
                ret = lambda: MixerSpec(type="retention", decay=[1 - 2.0 ** (-5 - i % 4) for i in range(zs["ret"]["heads"])],
                                        rot=RotarySpec(dims=zs["ret"]["dim"], base=10000.0), moe=mo, **zs["ret"])
                lat = lambda: MixerSpec(type="latent_attention", scale=(zs["lat"]["dim"] + zs["lat"]["rot_dim"]) ** -0.5, rot=rot, moe=mo, **zs["lat"])
                layers = [lat(), ret(), lat(), ret()]
                cfg = Config(hidden_size=W, intermediate_size=0, vocab_size=vocab, num_hidden_layers=4, num_attention_heads=layers[0].heads,
                             num_key_value_heads=layers[0].heads, rms_norm_eps=1e-6, head_dim=128, max_seq_len=mseq, block_kind="setodra",
                             layers=layers, model_prefix="", embed_scale=1.0)
                sd = make_mixer_checkpoint(cfg, "bf16", seed=5, device=env.dev, std=0.02)
                r, la = zs["ret"], zs["lat"]
                n_ret = 2 * r["heads"] * r["dim"] + 2 * r["heads"] * r["vdim"]
                n_lat = la["heads"] * (la["dim"] + la["rot_dim"]) + la["kv_rank"] + la["rot_dim"]
                ff_act = mo.top * mo.ff + mo.shared_ff
                lat_up = 2.0 * la["heads"] * la["kv_rank"] * (la["dim"] + la["vdim"])
                lin = 2 * 2.0 * W * (n_ret + r["heads"] * r["vdim"]) + 2 * (2.0 * W * (n_lat + la["heads"] * la["vdim"]) + lat_up)
                flop_tok = lin + 4 * (2.0 * W * 3 * ff_act + 2.0 * W * (mo.experts + mo.identity)) + 2 * 4.0 * r["heads"] * r["dim"] * r["vdim"]
                att_flops = lambda S: 2 * 2.0 * la["heads"] * (2 * la["kv_rank"] + la["rot_dim"]) * (S * (S + 1) // 2)
                wbytes = lin + 4 * (2.0 * W * 3 * ff_act)
                state_bytes = 2 * 8.0 * r["heads"] * r["dim"] * r["vdim"] + 2 * 2.0 * ctx_len * (la["kv_rank"] + la["rot_dim"])
            t = _time_listed_model(env, cfg, sd, batch, seq, ctx_len, steps, reps, mseq)
            del sd
            torch.cuda.empty_cache()
            launches += t["launches"]
            M, ms, dms = batch * seq, t["prefill"]["ms"], t["decode"]["ms_per_token"]
            flops = flop_tok * M + batch * att_flops(seq) + 2.0 * batch * vocab * W
            dbytes = wbytes + state_bytes + 2.0 * vocab * W
            row[arch] = {"prefill": {"tok_s": M / (ms / 1e3), "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
                                     "frac_of_tensor_peak": flops / (ms * 1e-3) / 1e12 / pk["tc"], "finite": t["prefill"]["finite"]},
                         "decode": {"tok_s": 1e3 / dms, "ms_per_token": dms, "gb_s": dbytes / (dms * 1e-3) / 1e9,
                                    "frac_of_hbm_peak": dbytes / (dms * 1e-3) / 1e9 / pk["hbm"], "launches_per_token": t["decode"]["launches_per_token"],
                                    "finite": t["decode"]["finite"]}}
        row["prefill_ratio"] = row["nuvarax"]["prefill"]["tok_s"] / row["closest"]["prefill"]["tok_s"]
        row["decode_ratio"] = row["nuvarax"]["decode"]["tok_s"] / row["closest"]["decode"]["tok_s"]
        out[name] = row
    head = out[sizes[-1]]
    return {"metric": f"nuvarax prefill tok/s (4 layers, width {head['size']['width']}, bf16, bs={batch} x {seq})", "value": head["nuvarax"]["prefill"]["tok_s"],
            "unit": "tok/s", "ms_per_step": head["nuvarax"]["prefill"]["ms"], "steps": reps, "warmup": 1, "gpu_launches": int(launches),
            "config": {"workload": f"Nuvarax vs Setodra at equal width, layer count and active feed-forward width, 4 layers, bf16, prefill bs={batch} x {seq}, "
                                   f"decode bs=1 at {ctx_len} context x {steps} steps", "l2": "prefill activations / decode weights exceed L2"},
            "peaks": {"tensor_tflops": pk["tc"], "hbm_gbs": pk["hbm"], "source": pk["src"]}, "sizes": out}


NETOLORN_SIZES = {  # layer sizes of real models (random weights): sink attention + dense feed-forward, windowed latent attention + routed feed-forward
    "1k": dict(width=1024, ff=4224, window=1024, keep_first=4, side=128,
               att=dict(heads=8, kv_heads=2, dim=128, vdim=128, rot_dims=64),
               lat=dict(heads=8, dim=128, vdim=128, q_rank=384, kv_rank=512), moe=dict(experts=32, top=4, ff=704, shared_ff=1408)),
    "2k": dict(width=2048, ff=11264, window=1024, keep_first=4, side=128,
               att=dict(heads=16, kv_heads=4, dim=128, vdim=128, rot_dims=64),
               lat=dict(heads=16, dim=128, vdim=128, q_rank=768, kv_rank=512), moe=dict(experts=64, top=6, ff=1408, shared_ff=2816)),
}


def netolorn_leg(env: Env, sizes=("1k", "2k"), batch: int = 4, seq: int = 4096, ctx_len: int = 2048, steps: int = 32, reps: int = 3) -> dict:
    """`--workload netolorn`: the Netolorn design (mixer-list blocks with squashing norms on both sides of every sublayer and a
    per-layer token input) in three 4-layer models per size, each beside the framework's closest existing model at equal width:
      attention   4 x (grouped-query attention with a partial rotation, unit-RMS q / k, a window that keeps the first tokens, a sink
                  and an output gate + dense feed-forward)  beside Nigenex (windowed grouped-query attention + dense feed-forward)
      latent      4 x (windowed latent attention without positions + routed clamped feed-forward with a shared expert)  beside the
                  Setodra-style latent attention layer (+ routed feed-forward of the same sizes)
      mixed       attention, latent, attention, latent (the headline number; no counterpart)
    all through TextModelBase / forward_batch.  Workload and timing as in the Setodra leg."""
    import torch
    from cake_b200.config import Config, LayerSpec, MixerSpec, MoeSpec, RotarySpec
    from cake_b200.synth import make_listed_checkpoint, make_mixer_checkpoint, make_netolorn_checkpoint
    pk = peaks()
    out, launches, vocab = {}, 0, 32768
    mseq = max(seq, ctx_len + steps + 8)
    for name in sizes:
        z = NETOLORN_SIZES[name]
        W, ff, win, keep, side, a, la, mo = z["width"], z["ff"], z["window"], z["keep_first"], z["side"], z["att"], z["lat"], z["moe"]
        ff_act = mo["top"] * mo["ff"] + mo["shared_ff"]
        keys_win = lambda S: sum(min(i + 1, win) for i in range(S))
        keys_kept = lambda S: sum(min(keep, max(0, i + 1 - win)) for i in range(S))
        att_layer = {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
                     "mixer": {"heads": a["heads"], "kv_heads": a["kv_heads"], "dim": a["dim"], "vdim": a["vdim"], "scale": a["dim"] ** -0.5,
                               "mask": {"size": win, "keep_first": keep},
                               "rot": {"dims": a["rot_dims"], "base": 10000.0, "scaling": {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}}
        lat_layer = {"type": "latent_attention",
                     "mlp": {"kind": "moe", "router": {"experts": mo["experts"], "top": mo["top"]}, "expert": {"ff": mo["ff"], "limit": 7.0},
                             "shared": {"ff": mo["shared_ff"], "limit": 7.0}},
                     "mixer": {"heads": la["heads"], "dim": la["dim"], "vdim": la["vdim"], "q_rank": la["q_rank"], "kv_rank": la["kv_rank"],
                               "scale": la["dim"] ** -0.5, "mask": {"size": win}}}
        # algorithmic work per token and layer: products [flops], weights read by one decoded token [bytes], cache rows read [bytes]
        Ha, Ga, Hl, R = a["heads"], a["kv_heads"], la["heads"], la["kv_rank"]
        side_f = 2.0 * W * 2 * side
        att_lin = 2.0 * W * (Ha * a["dim"] + Ga * (a["dim"] + a["vdim"]) + 2 * Ha * a["vdim"]) + 2.0 * W * 3 * ff + side_f
        lat_lin = (2.0 * W * (la["q_rank"] + R + Hl + Hl * la["vdim"]) + 2.0 * la["q_rank"] * Hl * la["dim"] + 2.0 * Hl * R * (la["dim"] + la["vdim"])
                   + 2.0 * W * 3 * ff_act + 2.0 * W * (mo["experts"] + 1) + side_f)
        att_key, lat_key = 2.0 * Ha * (a["dim"] + a["vdim"]), 2.0 * Hl * 2 * R
        att_cache = 2.0 * Ga * (a["dim"] + a["vdim"]) * (min(win, ctx_len) + keep)
        lat_cache = 2.0 * R * min(win, ctx_len)
        row = {"size": z}
        for arch in ("attention", "attention_closest", "latent", "latent_closest", "mixed"):
            if arch in ("attention", "latent", "mixed"):
                order = {"attention": [att_layer] * 4, "latent": [lat_layer] * 4, "mixed": [att_layer, lat_layer, att_layer, lat_layer]}[arch]
                cfg = Config.from_hf({"architecture": "Netolorn", "width": W, "vocab": vocab, "norm": {"eps": 1e-6}, "token_side": {"dim": side}, "layers": order})
                cfg.max_seq_len = mseq
                sd = make_netolorn_checkpoint(cfg, "bf16", seed=5, device=env.dev, std=0.02)
                n_att = sum(1 for L in order if L["type"] == "attention")
                flop_tok = n_att * att_lin + (4 - n_att) * lat_lin
                att_flops = lambda S, n_att=n_att: (n_att * att_key + (4 - n_att) * lat_key) * keys_win(S) + n_att * att_key * keys_kept(S)
                dbytes = flop_tok + n_att * att_cache + (4 - n_att) * lat_cache   # a weight is read once per decoded token: 2 bytes = 2 flops
            elif arch == "attention_closest":
                spec = LayerSpec(heads=Ha, kv_heads=Ga, head_dim=a["dim"], window=win, scale=a["dim"] ** -0.5, softcap=30.0, ff=ff)
                cfg = Config(hidden_size=W, intermediate_size=ff, vocab_size=vocab, num_hidden_layers=4, num_attention_heads=Ha, num_key_value_heads=Ga,
                             head_dim=a["dim"], max_seq_len=mseq, block_kind="nigenex", layers=[spec] * 4, logit_softcap=30.0, model_prefix="")
                sd = make_listed_checkpoint(cfg, "bf16", seed=5, device=env.dev, std=0.02)
                flop_tok = 4 * 2.0 * W * ((Ha + Ga) * a["dim"] + Ha + 3 * ff + Ha * a["dim"])
                att_flops = lambda S: 4 * 4.0 * Ha * a["dim"] * keys_win(S)
                dbytes = flop_tok + 4 * 2.0 * Ga * a["dim"] * min(win, ctx_len)
            else:
                rd = 64
                m = MoeSpec(scale=2.5, experts=mo["experts"], identity=0, top=mo["top"], ff=mo["ff"], shared_ff=mo["shared_ff"])
                rot = RotarySpec(dims=rd, base=10000.0, factor=8.0, fast=32.0, slow=1.0, original=2048)
                lat = lambda: MixerSpec(type="latent_attention", scale=(la["dim"] + rd) ** -0.5, rot=rot, moe=m, heads=Hl, dim=la["dim"], rot_dim=rd,
                                        vdim=la["vdim"], kv_rank=R)
                layers = [lat(), lat(), lat(), lat()]
                cfg = Config(hidden_size=W, intermediate_size=0, vocab_size=vocab, num_hidden_layers=4, num_attention_heads=Hl, num_key_value_heads=Hl,
                             rms_norm_eps=1e-6, head_dim=128, max_seq_len=mseq, block_kind="setodra", layers=layers, model_prefix="", embed_scale=1.0)
                sd = make_mixer_checkpoint(cfg, "bf16", seed=5, device=env.dev, std=0.02)
                n_lat = Hl * (la["dim"] + rd) + R + rd
                flop_tok = 4 * (2.0 * W * (n_lat + Hl * la["vdim"]) + 2.0 * Hl * R * (la["dim"] + la["vdim"]) + 2.0 * W * 3 * ff_act + 2.0 * W * mo["experts"])
                att_flops = lambda S: 4 * 2.0 * Hl * (2 * R + rd) * (S * (S + 1) // 2)   # no window: every earlier latent row
                dbytes = flop_tok + 4 * 2.0 * ctx_len * (R + rd)
            t = _time_listed_model(env, cfg, sd, batch, seq, ctx_len, steps, reps, mseq)
            del sd
            torch.cuda.empty_cache()
            launches += t["launches"]
            M, ms, dms = batch * seq, t["prefill"]["ms"], t["decode"]["ms_per_token"]
            flops = flop_tok * M + batch * att_flops(seq) + 2.0 * batch * vocab * W
            dbytes += 2.0 * vocab * W
            row[arch] = {"prefill": {"tok_s": M / (ms / 1e3), "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
                                     "frac_of_tensor_peak": flops / (ms * 1e-3) / 1e12 / pk["tc"], "finite": t["prefill"]["finite"],
                                     "launches": t["prefill"]["launches"]},
                         "decode": {"tok_s": 1e3 / dms, "ms_per_token": dms, "gb_s": dbytes / (dms * 1e-3) / 1e9,
                                    "frac_of_hbm_peak": dbytes / (dms * 1e-3) / 1e9 / pk["hbm"], "launches_per_token": t["decode"]["launches_per_token"],
                                    "finite": t["decode"]["finite"]}}
        for kind in ("attention", "latent"):   # how far from the roofline each is, the new design over the closest model (1 = equally far)
            row[kind + "_prefill_distance"] = row[kind + "_closest"]["prefill"]["frac_of_tensor_peak"] / row[kind]["prefill"]["frac_of_tensor_peak"]
            row[kind + "_decode_distance"] = row[kind + "_closest"]["decode"]["frac_of_hbm_peak"] / row[kind]["decode"]["frac_of_hbm_peak"]
        out[name] = row
    head = out[sizes[-1]]
    return {"metric": f"netolorn prefill tok/s (4 layers, width {head['size']['width']}, bf16, bs={batch} x {seq})", "value": head["mixed"]["prefill"]["tok_s"],
            "unit": "tok/s", "ms_per_step": head["mixed"]["prefill"]["ms"], "steps": reps, "warmup": 1, "gpu_launches": int(launches),
            "config": {"workload": f"Netolorn (attention / latent / mixed layer orders) vs Nigenex and the Setodra latent layer at equal width, 4 layers, bf16, "
                                   f"prefill bs={batch} x {seq}, decode bs=1 at {ctx_len} context x {steps} steps",
                       "l2": "prefill activations / decode weights exceed L2"},
            "peaks": {"tensor_tflops": pk["tc"], "hbm_gbs": pk["hbm"], "source": pk["src"]}, "sizes": out}


# ------------------------------------------------------------------------------------------------
def run_cuda(args):
    env = Env(args)
    K, W = args.steps, max(args.warmup, 3)
    world, rank = env.world, env.rank
    extras = args.extras
    if args.workload == "nigenex":
        if rank == 0:
            if env.sampler:
                env.sampler.start()
            line = nigenex_leg(env, sizes=tuple(args.sizes.split(",")), steps=max(4, min(args.steps, 64)))
            line["clocks"] = env.sampler.stop() if env.sampler else None
            line.update({"n_gpus": 1, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic"})
            emit(line)
        return
    if args.workload == "setodra":
        if rank == 0:
            if env.sampler:
                env.sampler.start()
            sizes = tuple((args.sizes if args.sizes != "2k,4k,4k-hd64" else "1k,2k").split(","))
            line = setodra_leg(env, sizes=sizes, batch=args.pf_batch, seq=args.pf_seq, steps=max(4, min(args.steps, 64)))
            line["clocks"] = env.sampler.stop() if env.sampler else None
            line.update({"n_gpus": 1, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic"})
            emit(line)
        return
    if args.workload == "nuvarax":
        if rank == 0:
            if env.sampler:
                env.sampler.start()
            sizes = tuple((args.sizes if args.sizes != "2k,4k,4k-hd64" else "1k,2k").split(","))
            line = nuvarax_leg(env, sizes=sizes, batch=args.pf_batch, seq=args.pf_seq, steps=max(4, min(args.steps, 64)))
            line["clocks"] = env.sampler.stop() if env.sampler else None
            line.update({"n_gpus": 1, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic"})
            emit(line)
        return
    if args.workload == "netolorn":
        if rank == 0:
            if env.sampler:
                env.sampler.start()
            sizes = tuple((args.sizes if args.sizes != "2k,4k,4k-hd64" else "1k,2k").split(","))
            line = netolorn_leg(env, sizes=sizes, batch=args.pf_batch, seq=args.pf_seq, steps=max(4, min(args.steps, 64)))
            line["clocks"] = env.sampler.stop() if env.sampler else None
            line.update({"n_gpus": 1, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic"})
            emit(line)
        return
    if args.workload == "prefill":
        if rank == 0:
            line = prefill_leg(env, reps=max(1, min(args.steps, 5)))
            line.update({"n_gpus": 1, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic"})
            emit(line)
        return
    parity = not args.no_parity and args.model == "8b"
    line = decode_leg(env, args.model, K, W, args.e2e_steps, parity=parity, isolated=(world == 1 and not args.no_isolated),
                      cpu_leg=(world == 1 and not args.no_cpu))
    # ---- further BASELINE configs riding on the same line -------------------------------------------------------
    if extras != "none" and args.model == "8b":
        if world == 8 or (extras == "all" and world > 1):
            guard = threading.Timer(420.0, lambda: (rank == 0 and emit(line), os._exit(0)))
            guard.daemon = True
            guard.start()       # a hung 70B leg must not cost the 8B line
            try:
                c3 = decode_leg(env, "70b", min(K, 32), 3, 0, parity=False, isolated=False, cpu_leg=False)
                if rank == 0:
                    pk = peaks()
                    line["config3"] = {k: c3[k] for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "config",
                                                          "gpu_launches", "token_roofline", "tokens_sha", "steps_trace") if k in c3}
                    line["config3"]["frac_of_single_stream_ceiling"] = c3["value"] / c3["token_roofline"]["roofline_tok_s_single_stream"]
            except Exception as e:  # noqa: BLE001
                if rank == 0:
                    line["config3"] = {"error": str(e)}
            guard.cancel()
        if world == 1 and rank == 0:
            try:  # 139 GB of bf16 weights + KV fit one 180 GB B200: the 70B model without the pipeline (context for config3)
                c3 = decode_leg(env, "70b", min(K, 16), 3, 4, parity=False, isolated=False, cpu_leg=False)
                line["config3_one_gpu"] = {k: c3[k] for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "config", "e2e",
                                                              "gpu_launches", "roofline", "token_roofline", "tokens_sha") if k in c3}
                line["config3_one_gpu"]["frac_of_single_stream_ceiling"] = c3["value"] / c3["token_roofline"]["roofline_tok_s_single_stream"]
            except Exception as e:  # noqa: BLE001
                line["config3_one_gpu"] = {"error": f"{type(e).__name__}: {e}"}
            for name, fn in (("config0", config0_leg), ("config4", prefill_leg)):
                try:
                    line[name] = fn(env)
                except Exception as e:  # noqa: BLE001
                    line[name] = {"error": f"{type(e).__name__}: {e}"}
    if rank == 0:
        emit(line)
    if env.sampler:
        env.sampler.close()
    if world > 1:
        env.dist.barrier()
        env.dist.destroy_process_group()


_REAL_STDOUT = None


def quiet_stdout():
    """The contract is ONE JSON line on stdout.  Libraries print there too (NCCL's version banner, warnings): route fd 1
    to stderr for the whole run and keep a private handle for the result line."""
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def emit(line: dict):
    out = _REAL_STDOUT or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--model", default="8b", choices=["8b", "70b"])
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "nigenex", "setodra", "nuvarax", "netolorn"])
    ap.add_argument("--pf-batch", type=int, default=4, help="--workload setodra / nuvarax / netolorn: batch rows of the prefill step")
    ap.add_argument("--pf-seq", type=int, default=4096, help="--workload setodra / nuvarax / netolorn: tokens per row of the prefill step")
    ap.add_argument("--sizes", default="2k,4k,4k-hd64", help="--workload nigenex: which of NIGENEX_SIZES to run")
    ap.add_argument("--extras", default="auto", choices=["auto", "none", "all"],
                    help="auto: config0 + config4 at N=1, config3 (70B) at N=8; none: the headline only")
    ap.add_argument("--e2e-steps", type=int, default=64)
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the first tokens")
    ap.add_argument("--no-isolated", action="store_true", help="skip the stand-alone per-op kernel timings")
    args = ap.parse_args()
    quiet_stdout()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
