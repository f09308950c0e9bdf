#!/usr/bin/env python
"""Prefill throughput of the 1B-class Complexity model (bf16) on B200 (the headline metric)
through the drop-in ``ComplexityModel`` API of this repository.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # CPU arm: the oracle port on the host cores

One step = one forward pass to logits over this rank's share of the global batch
(32 sequences x 2048 tokens, split data-parallel across ranks; no collective on the data
path).  Rank 0 prints ONE JSON line.
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

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "prefill tokens/s (1B bf16)"
UNIT = "tokens/s"
WORKLOAD = "1B-class prefill: hidden 2048, 24 layers, 16Q/8KV (D 128), intermediate 5632, " \
           "8 experts + shared, mu guidance, vocab 32000, batch 32 x seq 2048 Zipf(1.1) ids"
MODEL = dict(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=24,
             num_attention_heads=16, num_key_value_heads=8, num_experts=8)
GLOBAL_BATCH, SEQ_LEN = 32, 2048
# DRAM traffic of one cd_mu_qkv launch per token, from an ncu small-case capture of the kernel
# (dram__bytes_read + dram__bytes_write = 555 + 182 MB at 24 576 tokens)
MU_QKV_DRAM_BYTES_PER_TOKEN = 737.46e6 / 24576


def zipf_probabilities(vocab_size: int, s: float) -> torch.Tensor:
    """p(rank r) proportional to r^-s over ranks 1..V; token id = rank - 1."""
    p = torch.arange(1, vocab_size + 1, dtype=torch.float64).pow(-s)
    return p / p.sum()


def zipf_token_ids(vocab_size: int, s: float, count: int, seed: int = 0) -> torch.Tensor:
    """`count` synthetic token ids drawn from the Zipf law with a seeded CPU generator."""
    g = torch.Generator().manual_seed(seed)
    return torch.multinomial(zipf_probabilities(vocab_size, s).float(), count, replacement=True,
                             generator=g)


def shard_batch(global_batch: int, world: int, rank: int):
    """Contiguous split of the batch rows across ranks (sizes differ by at most one)."""
    base, extra = divmod(global_batch, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def aggregate_ms(local_ms: float, dist=None, device=None) -> float:
    """Step time of the whole job: the MAX over ranks of the device-measured time."""
    t = torch.tensor([local_ms], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def flops_per_token(cfg: dict, seq_len: int) -> dict:
    """Algorithmic FLOPs per token of each GEMM entry point (per layer unless noted)."""
    H, V, L = cfg["hidden_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    I_e = cfg["intermediate_size"] // cfg["num_experts"]
    D = H // cfg["num_attention_heads"]
    q_dim, kv_dim = cfg["num_attention_heads"] * D, cfg["num_key_value_heads"] * D
    return {
        "mu_qkv": 2 * 2 * H * (q_dim + 2 * kv_dim),
        "linear_o_proj": 2 * q_dim * H,
        "moe_up_routed": 4 * H * I_e,
        "moe_up_shared": 4 * H * I_e,
        "moe_down": 2 * H * (2 * I_e),
        "mu_proj": 2 * H * H,
        "linear_lm_head": 2 * H * V,          # once per token, not per layer
        "attention": 4 * seq_len * q_dim // 2,
        "layers": L,
    }


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "hbm_gbs": d["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0,
            "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs: NVML from a
    thread of this process (no start-up delay, so short regions still get samples), nvidia-smi
    as the fallback."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20,
                   "hw_thermal_slowdown": 0x40}
    _nvml_ready = False

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None
        self.samples, self.mask, self.max_mhz = [], 0, None
        self.handle, self.stop_flag, self.thread = None, threading.Event(), None
        try:
            import pynvml
            if not ClockSampler._nvml_ready:
                pynvml.nvmlInit()
                ClockSampler._nvml_ready = True
            uuid = str(torch.cuda.get_device_properties(index).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.nvml = pynvml
        except Exception:
            self.handle = None

    def _poll(self):
        nv = self.nvml
        while not self.stop_flag.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                self.mask |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
            except Exception:
                pass
            self.stop_flag.wait(0.01)

    def start(self):
        if self.handle is not None:
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=1.0)
            if not self.samples:
                return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no samples"]}
            reasons = [n for n, bit in self.REASON_BITS.items() if self.mask & bit]
            return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                    "samples": len(self.samples), "reasons": sorted(reasons), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for r in self.rows if len(r) == 6 and r[0].isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in rows)]
        return {"sm_mhz": statistics.median(int(r[0]) for r in rows),
                "sm_max_mhz": int(rows[0][1]), "samples": len(rows), "reasons": reasons,
                "source": "nvidia-smi"}


# ------------------------------------------------------------------------------- our arm
def build_model(device):
    from complexity_deep_b200 import TokenRoutedMLP
    from complexity_deep_b200.models import ComplexityConfig, ComplexityModel
    torch.manual_seed(0)
    with torch.device(device):
        model = ComplexityModel(ComplexityConfig(**MODEL))
    model = model.to(dtype=torch.bfloat16).eval()
    table = TokenRoutedMLP._build_token_mapping(
        MODEL["vocab_size"], MODEL["num_experts"], zipf_probabilities(MODEL["vocab_size"], 1.1).float())
    with torch.no_grad():
        for layer in model.layers:
            layer.mlp.token_to_expert.copy_(table)
    return model


def run_ours(args):
    from complexity_deep_b200 import ops
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    model = build_model(dev)
    batch = args.batch or GLOBAL_BATCH
    lo, hi = shard_batch(batch, world, rank)
    n_local = hi - lo
    if args.expert_parallel:
        # tokens stay data-parallel, the 8 routed experts of every layer are sharded over the
        # ranks (not the headline configuration, which replicates the weights)
        if dist is None:
            raise SystemExit("--expert-parallel needs more than one GPU")
        table = model.layers[0].mlp.token_to_expert.cpu()
        load = torch.bincount(table, weights=zipf_probabilities(MODEL["vocab_size"], 1.1),
                              minlength=MODEL["num_experts"])
        model.enable_expert_parallel(exchange=args.ep_exchange, expert_load=load,
                                     max_tokens_per_rank=n_local * SEQ_LEN)
    steps_total = args.warmup + args.steps
    # a different id batch per step, all drawn up front on the host (seeded), pinned
    host_ids = [zipf_token_ids(MODEL["vocab_size"], 1.1, batch * SEQ_LEN, seed=s)
                .view(batch, SEQ_LEN)[lo:hi].contiguous().pin_memory() for s in range(steps_total)]
    dev_ids = [h.to(dev) for h in host_ids]
    host_next = torch.empty(n_local, dtype=torch.int64).pin_memory()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    @torch.no_grad()
    def step_device(i):
        return model(dev_ids[i]).logits

    graph = None
    if args.graph and not args.expert_parallel:
        # the end-to-end loop replays a CUDA graph of the forward (PrefillGraph is the serving
        # entry point of this package); if capture is not possible the eager call is timed
        try:
            from complexity_deep_b200.models import PrefillGraph
            graph = PrefillGraph(model, n_local, SEQ_LEN)
        except Exception as exc:  # noqa: BLE001
            print(f"[bench] CUDA-graph capture failed ({exc}); timing the eager call", file=sys.stderr)
            torch.cuda.synchronize()
            graph = None

    @torch.no_grad()
    def step_e2e(i):
        ids = host_ids[i].to(dev, non_blocking=True)
        logits = graph(ids) if graph is not None else model(ids).logits
        host_next.copy_(logits[:, -1, :].argmax(-1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return host_next

    def timed(step_fn, instrument):
        for i in range(args.warmup):
            step_fn(i)
        barrier()
        sampler = ClockSampler(local_rank)
        sampler.start()
        ops.PROFILE.reset(enabled=instrument)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(args.warmup, steps_total):
            step_fn(i)
        t1.record()
        barrier()
        ms = aggregate_ms(t0.elapsed_time(t1), dist, dev)
        clocks = sampler.stop()
        prof = ops.PROFILE.collect()
        ops.PROFILE.reset(enabled=False)
        return ms, clocks, prof

    # 1. eager forward with CUDA events around every kernel entry point (roofline, breakdown)
    ms_eager, clocks_eager, prof = timed(step_device, instrument=True)
    # 2. the same forward replayed from its CUDA graph, ids resident on the device -> `value`
    if graph is not None:
        @torch.no_grad()
        def step_graph(i):
            return graph(dev_ids[i])
        ms_dev, clocks, _ = timed(step_graph, instrument=False)
    else:
        ms_dev, clocks = ms_eager, clocks_eager
    # 3. end to end: ids from pinned host memory, next-token ids back to the host
    ms_e2e, clocks_e2e, _ = timed(step_e2e, instrument=False)
    ops.status_fetch()

    tokens_per_step = batch * SEQ_LEN
    value = tokens_per_step * args.steps / (ms_dev / 1e3)
    e2e = tokens_per_step * args.steps / (ms_e2e / 1e3)

    # roofline of the dominant GEMM entry point, from the events recorded in the timed region
    pk = peaks()
    fl = flops_per_token(MODEL, SEQ_LEN)
    local_tokens = n_local * SEQ_LEN
    kernels = {}
    for name, (launches, total_ms, kernel_launches) in prof.items():
        entry = {"launches": launches, "ms_total": round(total_ms, 3)}
        if name in fl:
            flop = fl[name] * local_tokens
            tf = flop / (total_ms / launches / 1e3) / 1e12
            entry.update(tflops=round(tf, 1), frac=round(tf / pk["bf16_tflops"], 4))
        kernels[name] = entry
    gemm_names = [n for n in kernels if n in fl]
    dom = max(gemm_names, key=lambda n: kernels[n]["ms_total"]) if gemm_names else None
    roofline = None
    if dom:
        k = kernels[dom]
        roofline = {"bound": "tensor", "kernel": "gemm_bf16_sm100_kernel", "entry": dom, "achieved": k["tflops"], "peak": pk["bf16_tflops"],
                    "peak_source": pk["source"] + " burst", "unit": "TFLOP/s", "frac": k["frac"],
                    "peak_sustained": pk["bf16_tflops_sustained"],
                    "frac_sustained": (round(k["tflops"] / pk["bf16_tflops_sustained"], 4)
                                       if pk["bf16_tflops_sustained"] else None),
                    "flop_per_launch": fl[dom] * local_tokens,
                    "ms_per_launch": round(k["ms_total"] / k["launches"], 4),
                    "traffic": (round(MU_QKV_DRAM_BYTES_PER_TOKEN * local_tokens)
                                if dom == "mu_qkv" else None),
                    "traffic_source": "ncu small-case capture: dram__bytes_read+write of "
                                      "cd_mu_qkv_rope at 24576 tokens (737 MB), scaled per token"}
    gpu_launches = sum(v[2] for v in prof.values())

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_dev / args.steps, 3),
        "ms_per_step_eager": round(ms_eager / args.steps, 3),
        "forward": ("CUDA-graph replay of ComplexityModel.forward (PrefillGraph); the `kernels` and "
                    "`roofline` entries come from the eager loop timed just before it"
                    if graph is not None else "eager ComplexityModel.forward"),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "b200",
        "config": {"workload": WORKLOAD, "global_batch": batch, "seq_len": SEQ_LEN,
                   "parallelism": (f"dp{world} tokens + ep{world} routed experts ({args.ep_exchange})"
                                   if args.expert_parallel else f"dp{world}"),
                   "tokens_per_gpu_per_step": local_tokens,
                   "l2": "no flush: per-step working set (3.2 GB weights, 268 MB per activation) >> 126 MB L2; new ids each step"},
        "e2e": {"value": round(e2e, 1), "unit": UNIT, "ms_per_step": round(ms_e2e / args.steps, 3),
                "h2d_bytes_per_step": n_local * SEQ_LEN * 8, "d2h_bytes_per_step": n_local * 8,
                "result": "next-token argmax of the last position of every sequence",
                "api": "PrefillGraph(model)(ids)" if graph is not None else "model(ids).logits"},
        "gpu_launches": gpu_launches,
        "clocks": clocks, "clocks_eager": clocks_eager, "clocks_e2e": clocks_e2e,
        "roofline": roofline, "kernels": kernels,
        "model_flops_utilisation": round(
            (sum(fl[k] for k in ("mu_qkv", "linear_o_proj", "moe_up_routed", "moe_up_shared",
                                 "moe_down", "mu_proj", "attention")) * fl["layers"]
             + fl["linear_lm_head"]) * value / world / 1e12 / pk["bf16_tflops"], 4),
    }
    if rank == 0 and world == 1 and not args.no_parity:
        line["parity"] = model_parity(model)
    # free the model before the layer workloads below
    del graph, model
    torch.cuda.empty_cache()
    if not args.no_layer_records:
        # The layer records are short measurements (tens of ms) quoted against the BURST peak, like
        # `bench.py --workload moe_layer / ep_layer` run alone.  Straight after the prefill loops the
        # GPUs are still in the power-capped state of a long run (and not all to the same degree,
        # which the layer's cross-GPU barriers then pay as skew): 7.0 instead of 5.6 ms per layer
        # measured on 4 GPUs.  A pause lets them leave that state; the record carries its SM clock.
        time.sleep(2.0)
        # second half of the metric, in the same run and process group: the isolated MoE layer on
        # one GPU, the expert-parallel scale-out layer (peer-store exchange) on several
        if world == 1:
            rec = layer_record(args, "moe_layer", dist, dev, rank, world, local_rank)
            line["moe_layer"] = compact_layer_record(rec)
        elif LAYER_CONFIGS["ep_layer"]["E"] % world == 0:
            rec = layer_record(args, "ep_layer", dist, dev, rank, world, local_rank)
            line["ep_layer"] = compact_layer_record(rec)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(sample_tokens=args.cpu_tokens, steps=2, warmup=1)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def compact_layer_record(rec: dict) -> dict:
    """The figures of a layer workload that travel inside the prefill line."""
    keep = ("value", "unit", "ms_per_step", "ms_per_step_eager", "forward", "replay_equals_eager",
            "ms_per_step_routing_cached",
            "tflops_routing_cached",
            "frac_of_peak", "frac_of_peak_routing_cached", "peak_source", "tokens_per_s", "parity",
            "rows_received_per_gpu", "clocks", "kernels")
    out = {k: rec[k] for k in keep if rec.get(k) is not None}
    out["config"] = {k: rec["config"][k] for k in ("workload", "T", "H", "E", "I_e", "I_s",
                                                   "parallelism", "tokens_per_gpu", "flop_per_step")}
    return out


@torch.no_grad()
def model_parity(model, tokens: int = 512) -> dict:
    """Logits of the benchmarked model itself (all 24 layers, its own weights) on one sequence
    of `tokens` Zipf ids against the fp32 oracle on the same bf16-rounded weights — a bounded
    sample the CPU finishes in seconds; causal attention makes a shorter sequence a sub-problem
    of the full one.  Figures only; the tests assert."""
    from complexity_deep_b200 import ops
    from oracle import complexity_oracle as oracle
    dev = next(model.parameters()).device
    ids = zipf_token_ids(MODEL["vocab_size"], 1.1, tokens, seed=12345).view(1, tokens)
    logits = model(ids.to(dev)).logits.float().cpu()
    ops.status_fetch()
    sd = {k: (v.float().cpu() if v.is_floating_point() else v.cpu())
          for k, v in model.state_dict().items()}
    ref, _ = oracle.model_forward(sd, MODEL, ids)
    del sd
    max_rel, mean_abs = oracle.error_metrics(logits, ref)
    return {"max_rel": float(f"{max_rel:.3e}"), "mean_abs": float(f"{mean_abs:.3e}"),
            "argmax_agreement": round(float((logits.argmax(-1) == ref.argmax(-1)).float().mean()), 4),
            "rms_ref": round(float(ref.pow(2).mean().sqrt()), 3),
            "bf16_rounding_of_exact_logits_mean_abs": float(
                f"{float((ref.to(torch.bfloat16).float() - ref).abs().mean()):.3e}"),
            "sample": f"logits of 1 x {tokens} tokens through all {MODEL['num_hidden_layers']} layers",
            "against": "fp32 oracle (CPU) on the same bf16-rounded weights",
            "tolerance": "max_rel <= 2e-2, mean_abs <= 2e-3"}


# ------------------------------------------------------------------------------- CPU arm
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


def load_reference_package():
    """The reference's own `complexity_deep` package from oracle/_ref (placed there, unmodified,
    by oracle/make_ref.py), or None.  It must win over this repository's import-name shim of
    the same name, so it goes first on the path and any earlier import is dropped."""
    if not os.path.isfile(os.path.join(REF_DIR, "complexity_deep", "__init__.py")):
        return None
    for name in [n for n in sys.modules if n == "complexity_deep" or n.startswith("complexity_deep.")]:
        del sys.modules[name]
    sys.path.insert(0, REF_DIR)
    try:
        import complexity_deep as ref
        if os.path.dirname(os.path.abspath(ref.__file__)) != os.path.join(REF_DIR, "complexity_deep"):
            return None
        return ref
    except Exception as exc:  # noqa: BLE001
        print(f"[bench] reference package in oracle/_ref failed to import ({exc})", file=sys.stderr)
        return None
    finally:
        sys.path.remove(REF_DIR)


def reference_model(ref, device, dtype):
    """The reference's ComplexityModel for the bench workload: its own constructor and
    initialisation under manual_seed(0), the bin-packed Zipf table copied into every layer."""
    from oracle import complexity_oracle as oracle
    torch.manual_seed(0)
    with torch.device(device):
        model = ref.ComplexityModel(ref.ComplexityConfig(**MODEL))
    model = model.to(dtype=dtype).eval()
    p = oracle.zipf_probabilities(MODEL["vocab_size"], 1.1).float()
    table = torch.from_numpy(oracle.build_token_mapping(MODEL["vocab_size"], MODEL["num_experts"], p))
    with torch.no_grad():
        for layer in model.layers:
            layer.mlp.token_to_expert.copy_(table)
    return model


def cpu_baseline(sample_tokens: int, steps: int, warmup: int) -> dict:
    """Times the reference's forward on the host cores, fp32, all threads, on one sequence of
    `sample_tokens` tokens of the same workload: the reference's own modules when oracle/_ref
    holds them (kind "reference"), else the oracle port (kind "port")."""
    from oracle import complexity_oracle as oracle
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = dict(MODEL)
    ref = load_reference_package()
    if ref is not None:
        model = reference_model(ref, "cpu", torch.float32)
        forward = lambda ids: model(ids).logits                      # noqa: E731
        kind, what = "reference", "the reference's own ComplexityModel (oracle/_ref, unmodified)"
    else:
        p = oracle.zipf_probabilities(cfg["vocab_size"], 1.1).float()
        cfg["token_to_expert"] = torch.from_numpy(
            oracle.build_token_mapping(cfg["vocab_size"], cfg["num_experts"], p))
        sd = oracle.random_model_state(cfg, seed=0, dtype=torch.float32)
        forward = lambda ids: oracle.model_forward(sd, cfg, ids)[0]  # noqa: E731
        kind, what = "port", "oracle port of the reference's PyTorch forward"
    times = []
    with torch.no_grad():
        for i in range(warmup + steps):
            ids = oracle.zipf_token_ids(cfg["vocab_size"], 1.1, sample_tokens, seed=i).view(1, -1)
            t = time.perf_counter()
            forward(ids)
            if i >= warmup:
                times.append(time.perf_counter() - t)
    total = sum(times)
    return {"value": round(sample_tokens * len(times) / total, 1), "unit": UNIT, "cores": cores,
            "kind": kind, "dtype": "f32", "seconds_per_step": round(total / len(times), 3),
            "sample": f"1 sequence x {sample_tokens} tokens of the same model (all 24 layers + lm_head), "
                      f"{what}, {cores} threads"}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    base = cpu_baseline(sample_tokens=args.cpu_tokens, steps=args.steps, warmup=args.warmup)
    line = {
        "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(base["seconds_per_step"] * 1e3, 1), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "impl": "reference",
        "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "seq_len": SEQ_LEN,
                   "parallelism": "host cores"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_reference_gpu(args):
    """Not part of the driver's contract: the UNMODIFIED reference (oracle/_ref) on one GPU in
    bf16, same workload and ids, CUDA events — the like-for-like figure for the kernels here."""
    ref = load_reference_package()
    if ref is None:
        print(json.dumps({"impl": "reference-gpu", "unavailable": "oracle/_ref is not populated "
                          "(run oracle/make_ref.py where the reference checkout is)"}), flush=True)
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    model = reference_model(ref, dev, torch.bfloat16)
    batch = args.batch or GLOBAL_BATCH
    steps_total = args.warmup + args.steps
    ids = [zipf_token_ids(MODEL["vocab_size"], 1.1, batch * SEQ_LEN, seed=s).view(batch, SEQ_LEN).to(dev)
           for s in range(steps_total)]
    with torch.no_grad():
        for i in range(args.warmup):
            model(ids[i])
        torch.cuda.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(args.warmup, steps_total):
            model(ids[i])
        t1.record()
        torch.cuda.synchronize()
    ms = t0.elapsed_time(t1)
    print(json.dumps({
        "metric": METRIC, "value": round(batch * SEQ_LEN * args.steps / (ms / 1e3), 1), "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True, "dtype": "bf16",
        "data": "synthetic", "impl": "reference-gpu",
        "config": {"workload": WORKLOAD, "global_batch": batch, "seq_len": SEQ_LEN,
                   "parallelism": "1 GPU, the reference's stock PyTorch path"},
        "clocks": sampler.stop()}), flush=True)


# ------------------------------------------------------------------------------- layer modes
LAYER_CONFIGS = {
    # isolated token-routed MLP layer on one GPU
    "moe_layer": dict(T=16384, H=2048, E=8, I_e=5632, I_s=5632, V=32000, zipf=1.1, qkv=None),
    # expert-parallel scale-out layer incl. fused mu-QKV (32 Q / 8 KV heads, D 128)
    "ep_layer": dict(T=65536, H=4096, E=32, I_e=2816, I_s=11008, V=100000, zipf=1.0, qkv=6144),
}


def init_dist(dev, rank, world, force=False):
    """torch.distributed over NCCL, one process per GPU (None on a single GPU unless forced)."""
    if world == 1 and not force:
        return None
    import torch.distributed as dist
    if not dist.is_initialized():
        if "MASTER_ADDR" not in os.environ:
            os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29577")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    return dist


def layer_record(args, workload, dist, dev, rank, world, local_rank):
    """Times one MoE-layer workload for args.steps steps and checks sampled rows of every
    rank's output against the fp32 oracle of the unsharded layer.  Returns the record."""
    import torch.nn as nn
    from complexity_deep_b200 import TokenRoutedMLP, ops
    from complexity_deep_b200.expert_parallel import ExpertParallelMoE
    from oracle import complexity_oracle as oracle
    cfg = LAYER_CONFIGS[workload]
    T, H, E, I_e, I_s, V = (cfg[k] for k in ("T", "H", "E", "I_e", "I_s", "V"))
    lo, hi = shard_batch(T, world, rank)
    t_loc = hi - lo
    torch.manual_seed(0)                                   # same weights on every rank
    p = zipf_probabilities(V, cfg["zipf"]).float()
    with torch.device(dev):
        mlp = TokenRoutedMLP(H, I_e * E, E, V, True, None)
        if I_s != I_e:   # shared expert wider than one routed expert: swap the three Linears
            mlp.shared_gate, mlp.shared_up = nn.Linear(H, I_s, bias=False), nn.Linear(H, I_s, bias=False)
            mlp.shared_down = nn.Linear(I_s, H, bias=False)
        for lin in (mlp.shared_gate, mlp.shared_up, mlp.shared_down):
            nn.init.normal_(lin.weight, 0.0, 0.02)
    mlp = mlp.to(torch.bfloat16).eval()
    table = TokenRoutedMLP._build_token_mapping(V, E, p)
    with torch.no_grad():
        mlp.token_to_expert.copy_(table)
    ep = None
    if workload == "ep_layer":
        # expected rows per expert from the token frequencies, for the balanced placement
        load = torch.bincount(table, weights=p.double(), minlength=E)
        ep = ExpertParallelMoE(mlp, expert_load=load if args.ep_placement == "balanced" else None,
                               exchange=args.ep_exchange, max_tokens_per_rank=t_loc + 64)
    steps_total = args.warmup + args.steps
    gen = torch.Generator(device=dev).manual_seed(1 + rank)
    x = torch.randn(t_loc, H, device=dev, generator=gen).to(torch.bfloat16)
    ids = [zipf_token_ids(V, cfg["zipf"], T, seed=s)[lo:hi].to(dev) for s in range(steps_total)]
    w_qkv = w_mu = mu_prev = None
    if cfg["qkv"]:
        w_qkv = (torch.randn(cfg["qkv"], H, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
        w_mu = (torch.randn(cfg["qkv"], H, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
        mu_prev = torch.randn(t_loc, H, device=dev, generator=gen).to(torch.bfloat16)

    @torch.no_grad()
    def step(i):
        if w_qkv is not None:
            ops.mu_qkv(x, mu_prev, w_qkv, w_mu)
        if ep is not None:
            return ep.forward(x.view(1, t_loc, H), ids[i].view(1, t_loc))
        return mlp(x.view(1, t_loc, H), ids[i].view(1, t_loc))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ops.PROFILE.reset(enabled=True)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(args.warmup, steps_total):
        step(i)
    t1.record()
    barrier()
    ms = aggregate_ms(t0.elapsed_time(t1), dist, dev)
    clocks = sampler.stop()
    prof = ops.PROFILE.collect()
    ops.PROFILE.reset(enabled=False)
    # The same steps replayed from a CUDA graph of the layer (dispatch, exchange plan and barriers
    # included: they all take their sizes from device memory), new ids copied into the captured
    # id buffer before every replay: the figure of the layer without the interpreter's launch
    # overhead, which with several processes per host otherwise shows up as skew at the layer's
    # first cross-GPU barrier.  All ranks take the replay or none does.
    ms_eager, forward = ms, "eager"
    y_replayed = None
    if args.graph:
        graph_ok = torch.ones(1, device=dev)
        g = None
        try:
            static_ids = ids[0].clone()

            @torch.no_grad()
            def step_static():
                if w_qkv is not None:
                    ops.mu_qkv(x, mu_prev, w_qkv, w_mu)
                if ep is not None:
                    return ep.forward(x.view(1, t_loc, H), static_ids.view(1, t_loc))
                return mlp(x.view(1, t_loc, H), static_ids.view(1, t_loc))

            static_ids.copy_(ids[1])          # a new version of the buffer: the capture includes the dispatch
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                y_static = step_static()
        except Exception as exc:              # noqa: BLE001 - any capture problem means the eager figure stands
            print(f"[bench] {workload}: CUDA-graph capture failed ({exc}); keeping the eager figure",
                  file=sys.stderr)
            graph_ok.zero_()
            g = None
        if dist is not None:
            dist.all_reduce(graph_ok, op=dist.ReduceOp.MIN)
        if bool(graph_ok.item() > 0) and g is not None:
            for i in range(args.warmup):
                static_ids.copy_(ids[i])
                g.replay()
            barrier()
            t0.record()
            for i in range(args.warmup, steps_total):
                static_ids.copy_(ids[i])
                g.replay()
            t1.record()
            barrier()
            ms = aggregate_ms(t0.elapsed_time(t1), dist, dev)
            forward = "cuda_graph_replay of the layer step, new ids copied into the captured buffer every step"
            y_replayed = y_static.clone()     # output of the last replay: ids[-1]
    # the same layer on an id batch whose dispatch (and exchange plan) is already cached, as
    # layers 2..L of a forward pass see it (three untimed steps first: the allocator's blocks
    # settle again after the graph replays, which live in their own pool)
    for _ in range(3):
        y = step(steps_total - 1)
    barrier()
    t0.record()
    for _ in range(args.steps):
        step(steps_total - 1)
    t1.record()
    barrier()
    ms_cached = aggregate_ms(t0.elapsed_time(t1), dist, dev)
    ops.status_fetch()
    # the replayed step and the eager step saw the same ids last: same bits expected
    replay_equal = None if y_replayed is None else bool(torch.equal(y_replayed, y))

    # parity: sampled rows of THIS rank's output against the fp32 oracle of the unsharded layer
    # on the same bf16-rounded weights and inputs; the worst rank is reported
    rows = torch.randperm(t_loc, generator=torch.Generator().manual_seed(7 + rank))[:96]
    sd = {k: v.detach().float().cpu() for k, v in mlp.named_parameters()}
    sd["token_to_expert"] = table
    with torch.no_grad():
        ref = oracle.token_routed_mlp(sd, "", x[rows.to(dev)].float().cpu()[None],
                                      ids[-1][rows.to(dev)].cpu()[None])[0]
    del sd
    max_rel, mean_abs = oracle.error_metrics(y.view(t_loc, H)[rows.to(dev)].float().cpu(), ref)
    worst = torch.tensor([max_rel, mean_abs], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    parity = {"max_rel": float(f"{worst[0].item():.3e}"), "mean_abs": float(f"{worst[1].item():.3e}"),
              "rows_per_gpu": int(rows.numel()), "rms_ref": round(float(ref.pow(2).mean().sqrt()), 3),
              "against": "fp32 oracle of the unsharded layer, worst rank",
              "within_tolerance": bool(worst[0].item() <= 2e-2 and worst[1].item() <= 2e-3 * max(
                  1.0, float(ref.pow(2).mean().sqrt())))}

    flop = 6 * T * H * I_e + 6 * T * H * I_s + (2 * T * 2 * H * cfg["qkv"] if cfg["qkv"] else 0)
    tflops = flop * args.steps / (ms / 1e3) / 1e12
    pk = peaks()
    received = None
    if ep is not None:
        rows_t = torch.tensor([ep.plan_for(ep.routing(ids[-1].view(1, t_loc)))[0].received],
                              device=dev)
        gathered = [torch.empty_like(rows_t) for _ in range(world)]
        dist.all_gather(gathered, rows_t)
        received = [int(r) for r in gathered]
    return {
        "metric": "MoE-layer TFLOP/s (bf16)", "value": round(tflops, 1), "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 4),
        "ms_per_step_eager": round(ms_eager / args.steps, 4), "forward": forward,
        "replay_equals_eager": replay_equal,
        "ms_per_step_routing_cached": round(ms_cached / args.steps, 4),
        "tflops_routing_cached": round(flop * args.steps / (ms_cached / 1e3) / 1e12, 1),
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "b200",
        "config": {"workload": workload, **{k: v for k, v in cfg.items()},
                   "parallelism": (f"ep{world}: {E // world} experts per GPU ({args.ep_placement} "
                                   f"placement, {args.ep_exchange} exchange), tokens dp{world}"
                                   if ep is not None else "1 GPU"),
                   "tokens_per_gpu": t_loc, "flop_per_step": flop},
        "tokens_per_s": round(T * args.steps / (ms / 1e3), 1),
        "frac_of_peak": round(tflops / world / pk["bf16_tflops"], 4),
        "frac_of_peak_routing_cached": round(flop * args.steps / (ms_cached / 1e3) / 1e12 / world
                                             / pk["bf16_tflops"], 4),
        "peak": pk["bf16_tflops"], "peak_source": pk["source"] + " burst, per GPU",
        "parity": parity,
        "rows_received_per_gpu": received, "clocks": clocks,
        "gpu_launches": sum(v[2] for v in prof.values()),
        "kernels": {k: {"launches": v[0], "ms_total": round(v[1], 3)} for k, v in prof.items()},
    }


def run_layer(args):
    """MoE-layer TFLOP/s: the isolated layer (1 GPU) or the expert-parallel layer (N GPUs, the
    T tokens split across ranks, experts sharded E/N per rank, exchange by peer stores or NCCL
    all-to-all)."""
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = init_dist(dev, rank, world, force=args.workload == "ep_layer")
    line = layer_record(args, args.workload, dist, dev, rank, world, local_rank)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_attention(args):
    """Prefill attention alone: cd_attention_prefill against torch SDPA (cuDNN) on the same
    buffer, 16 Q / 8 KV heads of 128 (the 1B configuration), kernel time from CUDA events."""
    import torch.nn.functional as F
    from complexity_deep_b200 import ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, S, hq, hkv, D = args.batch or 32, args.seq_len, 16, 8, 128
    g = torch.Generator(device=dev).manual_seed(0)
    qkv = torch.randn(B * S, (hq + 2 * hkv) * D, device=dev, generator=g).to(torch.bfloat16)
    q = qkv[:, :hq * D].view(B, S, hq, D).transpose(1, 2)
    k = qkv[:, hq * D:(hq + hkv) * D].view(B, S, hkv, D).transpose(1, 2)
    v = qkv[:, (hq + hkv) * D:].view(B, S, hkv, D).transpose(1, 2)
    fns = {"cd_attention_prefill": lambda: ops.attention_prefill(qkv, B, S, hq, hkv, D),
           "torch_sdpa": lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)}
    flop = 4 * B * hq * S * S * D / 2
    out = {}
    for name, fn in fns.items():
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            fn()
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / args.steps
        out[name] = {"ms": round(ms, 4), "tflops": round(flop / ms / 1e9, 1)}
    ops.status_fetch()
    a = fns["cd_attention_prefill"]().float().view(B, S, hq, D).transpose(1, 2)
    diff = float((a - fns["torch_sdpa"]().float()).abs().max())
    pk = peaks()
    print(json.dumps({"metric": "prefill attention TFLOP/s (bf16)", "value": out["cd_attention_prefill"]["tflops"],
                      "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                      "config": {"workload": "attn_prefill", "batch": B, "seq_len": S, "q_heads": hq,
                                 "kv_heads": hkv, "head_dim": D, "flop_per_launch": flop},
                      "kernels": out, "frac_of_peak": round(out["cd_attention_prefill"]["tflops"] / pk["bf16_tflops"], 4),
                      "max_abs_diff_vs_sdpa": diff, "dtype": "bf16", "data": "synthetic", "impl": "b200"}), flush=True)


def run_decode(args):
    """1B-class decode: concurrent sequences with a prefilled KV cache
    of 4096 tokens (values N(0,1) bf16), one new Zipf token per sequence per step, the new
    token attending to the whole cache.  The batch (256 sequences) is split data-parallel.
    Two timed loops over the same caches: the reference's calling convention (growing cache,
    all-zero additive mask) issued eagerly with events around every entry point -> `kernels`,
    `ms_per_step_eager`; and the fixed-launch step replayed from its CUDA graph
    (`DecodeGraph`) -> `value`, plus `e2e` with ids from pinned host memory and the argmax
    read back."""
    from complexity_deep_b200 import ops
    from complexity_deep_b200.core.attention import _KVBuffer
    from complexity_deep_b200.models import DecodeGraph
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    model = build_model(dev)
    batch = args.batch or 256
    lo, hi = shard_batch(batch, world, rank)
    B, P = hi - lo, args.cache_len
    cfg = MODEL
    D = cfg["hidden_size"] // cfg["num_attention_heads"]
    hkv, L = cfg["num_key_value_heads"], cfg["num_hidden_layers"]
    steps_total = args.warmup + args.steps
    gen = torch.Generator(device=dev).manual_seed(1 + rank)

    # one set of buffers serves both loops: the growing-cache loop appends in place into them
    dec = DecodeGraph(model, batch=B, capacity=P + steps_total + 8)
    for t in dec.cache.k + dec.cache.v:
        t.normal_(0.0, 1.0, generator=gen)

    def growing_view(buf):
        view = buf[:, :, :P]
        view._cd_kv = _KVBuffer(buf, P)
        return view

    ids = zipf_token_ids(cfg["vocab_size"], 1.1, batch * steps_total, seed=0).view(steps_total, batch)
    ids_host = ids[:, lo:hi].contiguous().pin_memory()
    ids = ids_host.to(dev)

    @torch.no_grad()
    def step_eager(i, past):
        kv_len = past[0][0].shape[2] + 1
        mask = torch.zeros(B, 1, 1, kv_len, dtype=torch.bfloat16, device=dev)
        out = model(ids[i].view(B, 1), attention_mask=mask, past_key_values=past, use_cache=True)
        return out.logits, out.past_key_values

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, instrument):
        for i in range(args.warmup):
            step_fn(i)
        barrier()
        sampler = ClockSampler(local_rank)
        sampler.start()
        ops.PROFILE.reset(enabled=instrument)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(args.warmup, steps_total):
            step_fn(i)
        t1.record()
        barrier()
        ms = aggregate_ms(t0.elapsed_time(t1), dist, dev)
        clocks = sampler.stop()
        prof = ops.PROFILE.collect() if instrument else {}
        ops.PROFILE.reset(enabled=False)
        ops.status_fetch()
        return ms, clocks, prof

    state = {"past": [(growing_view(k), growing_view(v)) for k, v in zip(dec.cache.k, dec.cache.v)]}

    def eager(i):
        _, state["past"] = step_eager(i, state["past"])

    ms_eager, _, prof = timed(eager, True)
    state.clear()

    dec.cache.set_length(P)
    ms, clocks, _ = timed(lambda i: dec.step(ids[i]), False)

    dec.cache.set_length(P)
    next_host = torch.empty(B, dtype=torch.int64).pin_memory()

    def step_e2e(i):
        logits = dec.step(ids_host[i].to(dev, non_blocking=True))
        next_host.copy_(logits[:, -1].argmax(-1), non_blocking=True)

    ms_e2e, _, _ = timed(step_e2e, False)

    H, V, E = cfg["hidden_size"], cfg["vocab_size"], cfg["num_experts"]
    I_e = cfg["intermediate_size"] // E
    nqkv = (cfg["num_attention_heads"] + 2 * hkv) * D
    weight_bytes = {  # bf16 weights one launch streams
        "mu_qkv": 2 * 2 * H * nqkv, "linear_o_proj": 2 * H * H, "moe_up_routed": 2 * 2 * E * H * I_e,
        "moe_up_shared": 2 * 2 * H * I_e, "moe_down": 2 * (E + 1) * H * I_e, "mu_proj": 2 * H * H,
        "linear_lm_head": 2 * H * V}
    pk = peaks()
    kernels = {}
    for name, (launches, total_ms, _) in prof.items():
        entry = {"launches": launches, "us_per_launch": round(total_ms / launches * 1e3, 2)}
        if name in weight_bytes:
            gbs = weight_bytes[name] / (total_ms / launches / 1e3) / 1e9
            entry.update(weight_gbs=round(gbs, 1), frac_of_hbm=round(gbs / pk["hbm_gbs"], 4))
        kernels[name] = entry
    cache_bytes = 2 * L * B * hkv * (P + steps_total / 2) * D * 2
    floor_w = sum(weight_bytes[k] * (L if k != "linear_lm_head" else 1) for k in weight_bytes)
    line = {
        "metric": "decode tokens/s (1B bf16)", "value": round(batch * args.steps / (ms / 1e3), 1),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 3),
        "ms_per_step_eager": round(ms_eager / args.steps, 3),
        "forward": "cuda_graph_replay (DecodeGraph); eager = growing cache + zero additive mask",
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "b200",
        "config": {"workload": f"1B-class decode, {batch} sequences, KV cache {P} tokens, whole cache attended",
                   "parallelism": f"dp{world}", "sequences_per_gpu": B},
        "e2e": {"value": round(batch * args.steps / (ms_e2e / 1e3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8,
                "api": "DecodeGraph(model, batch, capacity).step(ids)"},
        "hbm_floor_ms": {"weights": round(floor_w / pk["hbm_gbs"] / 1e6, 3),
                         "kv_cache": round(cache_bytes / pk["hbm_gbs"] / 1e6, 3)},
        "frac_of_hbm_floor": round((floor_w + cache_bytes) / pk["hbm_gbs"] / 1e6 / (ms / args.steps), 4),
        "clocks": clocks, "gpu_launches": sum(v[2] for v in prof.values()), "kernels": kernels,
    }
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference-gpu"])
    ap.add_argument("--batch", type=int, default=0, help="global batch override (debug only)")
    ap.add_argument("--cpu-tokens", type=int, default=2048,
                    help="tokens of the bounded CPU sample (one sequence)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the in-run oracle check of the logits")
    ap.add_argument("--no-layer-records", action="store_true",
                    help="prefill_1b: skip the MoE-layer (1 GPU) / expert-parallel layer (N GPUs) sub-record")
    ap.add_argument("--graph", dest="graph", action="store_true", default=True,
                    help="prefill_1b: the end-to-end loop replays a CUDA graph of the forward (default)")
    ap.add_argument("--no-graph", dest="graph", action="store_false")
    ap.add_argument("--expert-parallel", action="store_true",
                    help="prefill_1b: shard the routed experts over the ranks (extra, not the headline)")
    ap.add_argument("--ep-placement", default="balanced", choices=["balanced", "contiguous"],
                    help="ep_layer: which experts share a GPU")
    ap.add_argument("--ep-exchange", default="peer", choices=["peer", "nccl"],
                    help="ep_layer: peer stores from the kernels, or NCCL all-to-all")
    ap.add_argument("--cache-len", type=int, default=4096, help="decode_1b: prefilled KV tokens")
    ap.add_argument("--seq-len", type=int, default=SEQ_LEN, help="attn_prefill: sequence length")
    ap.add_argument("--workload", default="prefill_1b",
                    choices=["prefill_1b", "decode_1b", "attn_prefill"] + list(LAYER_CONFIGS),
                    help="prefill_1b is the headline; the layer modes report MoE-layer TFLOP/s")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "b200":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu(args)
    elif args.workload == "decode_1b":
        run_decode(args)
    elif args.workload == "attn_prefill":
        run_attention(args)
    elif args.workload != "prefill_1b":
        run_layer(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
