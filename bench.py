#!/usr/bin/env python
"""Benchmark of the MatMul-free LM inference hot path: HGRNBit-1.3B greedy decoding on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl ours|reference]

One "step" = one greedy decode step (all 24 layers, lm_head, arg-max) for the `--batch` sequences a GPU
holds.  With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank decodes its own
`--batch` sequences with a full replica of the packed weights and no collective on the data path (weak
scaling); the reported value is the tokens all ranks produce per second, timed on the device between
barriers, max over ranks.  Rank 0 prints ONE JSON line.

Inputs are synthetic (uniform random token ids) and weights are random-init N(0, 0.02), ternarised — there
is no network for checkpoints; model shape is the published 1.3B configuration.

`--impl reference` times the reference's own CPU path on the host cores, on a bounded sample of the same workload:
the reference package installed under baseline/_ref (or $MMFREELM_REFERENCE) with its five GPU-only leaves swapped for
the reference's own pure-PyTorch statements of the same math (RMSNorm -> rms_norm_ref, FusedRMSNormSwishGate ->
rms_norm_ref * o * sigmoid(o), FusedBitLinear -> BitLinear.forward, swiglu -> silu(x) * y, fused_recurrent_hgrn ->
naive_recurrent_hgrn); if that package cannot be imported, the restatement in oracle/mmfree_oracle.py stands in
(`cpu_baseline.kind` says which).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MODEL = dict(vocab_size=32000, hidden_size=2048, num_hidden_layers=24, intermediate_size=5632)
METRIC = "hgrnbit_1.3b_greedy_decode_tokens_per_s"
L2_BYTES = 126 * 1024 * 1024


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=32, help="sequences per GPU")
    ap.add_argument("--prompt", type=int, default=128, help="prompt tokens used to seed the recurrent state")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--layers", type=int, default=MODEL["num_hidden_layers"], help=argparse.SUPPRESS)
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary measurements (batch 1/256, prefill)")
    ap.add_argument("--eager", action="store_true",
                    help="decode step by step without the CUDA graph (for profiler launch lists; slower)")
    ap.add_argument("--skip-cpu", action="store_true", help="skip the CPU-baseline leg (for profiler runs)")
    ap.add_argument("--min-seconds", type=float, default=0.5,
                    help="the block of --steps steps is repeated until the timed region lasts at least this long")
    ap.add_argument("--throughput-steps", type=int, default=512,
                    help="decode steps of the multi-GPU 2.7B throughput measurement (N > 1 only)")
    return ap.parse_args()


def workload_name(args):
    return (f"HGRNBit-1.3B random-init ternarised, greedy decode, batch {args.batch} per GPU, "
            f"state seeded by a {args.prompt}-token prompt")


def config_dict(args, world):
    """The workload description both arms print (same keys, same values)."""
    return {"workload": workload_name(args), "per_gpu_batch": args.batch, "global_batch": world * args.batch,
            "parallelism": f"batch-sharded x{world}, no data-path collective",
            "l2_policy": "inputs larger than L2: one step streams 325 MB of packed weights (L2 = 126 MB)"}


# dram__bytes_read+write of one bitlinear_mma_kernel launch (M=32, K=2048, N=11264) from the profiler, per byte of
# packed weights that launch streams; DRAM traffic of this kernel is the weight stream plus the activation codes
NCU_DRAM_BYTES_PER_WEIGHT_BYTE = 5.883 / 5.767


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback (earlier measurement on this pool)"


# ----------------------------------------------------------------------------------------------------------
# clocks sampling during the timed region
# ----------------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------------------
# CPU arm: the reference algorithm on the host cores
# ----------------------------------------------------------------------------------------------------------
def load_reference():
    """The reference package itself (baseline/_ref or $MMFREELM_REFERENCE) made runnable on a CPU by swapping its five
    GPU-only leaves for the reference's own pure-PyTorch statements of the same math.  Returns its model classes, or
    None (with the reason) when the package is not importable here."""
    import warnings
    for cand in (os.environ.get("MMFREELM_REFERENCE"), str(ROOT / "baseline" / "_ref")):
        if cand and Path(cand, "mmfreelm").is_dir():
            break
    else:
        return None, "no reference package under baseline/_ref or $MMFREELM_REFERENCE"
    sys.dont_write_bytecode = True
    sys.path.insert(0, cand)
    try:
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            import torch.nn.functional as F
            import mmfreelm.layers.hgrn_bit as LAYER
            import mmfreelm.models.hgrn_bit.modeling_hgrn_bit as MODELING
            from mmfreelm.models import HGRNBitConfig, HGRNBitForCausalLM
            from mmfreelm.modules import fused_norm_gate as FNG
            from mmfreelm.modules import layernorm as LN
            from mmfreelm.ops import fusedbitnet as FB
            from mmfreelm.ops.hgrn.naive import naive_recurrent_hgrn
    except Exception as e:   # noqa: BLE001 - any import failure means "not available here"
        sys.path.remove(cand)
        return None, f"reference package not importable: {type(e).__name__}: {e}"

    def rms_fwd(self, x, residual=None, prenorm=False, residual_in_fp32=False):
        return LN.rms_norm_ref(x, self.weight, self.bias, residual=residual, eps=self.eps, prenorm=prenorm)

    def gate_fwd(self, x, o, residual=None, prenorm=False, residual_in_fp32=False):
        return FNG.rms_norm_ref(x, self.weight, self.bias, eps=self.eps) * o * torch.sigmoid(o)

    def sw(x, y):
        return F.silu(x) * y

    LN.RMSNorm.forward = rms_fwd
    FNG.FusedRMSNormSwishGate.forward = gate_fwd
    FB.FusedBitLinear.forward = FB.BitLinear.forward
    LAYER.swiglu = sw
    MODELING.swiglu = sw
    LAYER.fused_recurrent_hgrn = lambda x, g, initial_state=None, output_final_state=False: naive_recurrent_hgrn(
        x, g, initial_state, output_final_state)
    return (HGRNBitConfig, HGRNBitForCausalLM, FB.BitLinear), cand


def cpu_reference_step_time(batch: int, steps: int, warmup: int, budget_s: float):
    """Time one decode step (one new token per sequence, recurrent state carried) of the reference's CPU path.  A full
    1.3B step on CPU re-ternarises every weight (as the reference does on each call), so the sample is the first
    `n_layers` of the 24 layers plus the lm_head, and the step time is extrapolated linearly in the layer count;
    n_layers is chosen from a one- and two-layer calibration so that warmup + steps fit in `budget_s`.
    Returns (seconds per full step, threads, description of the sample, "reference" | "port")."""
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    ids = torch.randint(0, MODEL["vocab_size"], (batch, 1), generator=torch.Generator().manual_seed(0))
    ref, why = load_reference()

    if ref is not None:
        kind = "reference"
        HGRNBitConfig, HGRNBitForCausalLM, RefBitLinear = ref

        def build(n_layers):
            import warnings
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                model = HGRNBitForCausalLM(HGRNBitConfig(**{**MODEL, "num_hidden_layers": n_layers})).eval()
            g = torch.Generator().manual_seed(1234)
            with torch.no_grad():
                for m in model.modules():
                    if isinstance(m, RefBitLinear):
                        m.weight.normal_(0.0, 0.02, generator=g)
                model.model.embeddings.weight.normal_(0.0, 0.02, generator=g)
            return model

        def timed(model, n):
            ts = []
            with torch.no_grad():
                cache = model(input_ids=ids, use_cache=True).past_key_values          # first token builds the state
                for _ in range(n):
                    t0 = time.perf_counter()
                    out = model(input_ids=ids, past_key_values=cache, use_cache=True)
                    out.logits[:, -1].argmax(-1)
                    cache = out.past_key_values
                    ts.append(time.perf_counter() - t0)
            return ts
    else:
        kind = "port"
        from oracle import mmfree_oracle as O

        def build(n_layers):
            cfg = O.OracleConfig(**{**MODEL, "num_hidden_layers": n_layers})
            return O.OracleHGRNBit(cfg, O.random_weights(cfg, seed=0), dtype=torch.float32, linear="float")

        def timed(model, n):
            states = [torch.zeros(batch, 1, MODEL["hidden_size"]) for _ in range(model.cfg.num_hidden_layers)]
            ts = []
            for _ in range(n):
                t0 = time.perf_counter()
                logits, states = model.forward(ids, states, last_only=True)
                logits[:, -1].argmax(-1)
                ts.append(time.perf_counter() - t0)
            return ts

    m1, m2 = build(1), build(2)
    timed(m1, 1)
    t1 = min(timed(m1, 2))                       # one block + final norm + lm_head
    timed(m2, 1)
    t2 = min(timed(m2, 2))
    t_layer = max(t2 - t1, 1e-4)
    t_head = max(t1 - t_layer, 0.0)
    total_steps = steps + warmup
    n_layers = int(max(1, min(MODEL["num_hidden_layers"], (budget_s / total_steps - t_head) / t_layer)))
    model = m1 if n_layers == 1 else m2 if n_layers == 2 else build(n_layers)
    del m1, m2
    timed(model, warmup)
    ts = timed(model, steps)
    mean = sum(ts) / len(ts)
    per_layer = (mean - t_head) / n_layers
    full_step = t_head + per_layer * MODEL["num_hidden_layers"]
    what = ("the reference package itself (its GPU-only leaves swapped for its own pure-PyTorch math)" if kind == "reference"
            else f"the oracle restatement of the reference ({why})")
    sample = (f"{what}: batch {batch}, 1 new token, first {n_layers} of {MODEL['num_hidden_layers']} layers + lm_head in "
              f"fp32 (weight_quant re-evaluated per call as in the reference), {steps} steps; full-step time "
              f"extrapolated linearly in the layer count")
    return full_step, threads, sample, kind


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    full_step, threads, sample, kind = cpu_reference_step_time(args.batch, args.steps, args.warmup, budget_s=150.0)
    value = args.batch / full_step
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": full_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args, max(world, args.gpus)),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample,
                         "device": "host CPU (rank 0 only; the value is one host's throughput)"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------------------
def build_model(args, device, dtype=torch.bfloat16, spec=None):
    from matmulfreellm_b200.models import HGRNBitConfig, HGRNBitForCausalLM
    from matmulfreellm_b200.ops.fusedbitnet import BitLinear
    cfg = HGRNBitConfig(**(spec or {**MODEL, "num_hidden_layers": args.layers}))
    with torch.device(device):
        model = HGRNBitForCausalLM(cfg).eval()
    g = torch.Generator(device=device).manual_seed(1234)       # same weights on every rank
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, BitLinear):
                m.weight.normal_(0.0, 0.02, generator=g)
        model.model.embeddings.weight.normal_(0.0, 0.02, generator=g)
    model.pack_weights()
    return model.to(dtype)


def device_time_ms(fn, iters, stream):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(iters):
        fn()
    end.record(stream)
    end.synchronize()
    return start.elapsed_time(end) / iters


def median(xs):
    xs = sorted(xs)
    n = len(xs)
    return xs[n // 2] if n % 2 else 0.5 * (xs[n // 2 - 1] + xs[n // 2])


def multi_gpu_extras(args, device, rank, world, gen):
    """Only with N > 1 ranks: (a) a ragged batch generated sharded over the ranks and gathered with NCCL equals the same
    batch generated on one GPU; (b) the high-throughput configuration — HGRNBit-2.7B shapes, 64 sequences per GPU —
    decoded for --throughput-steps steps without any gather, with the step's tokens all-gathered on a side stream, and
    with the step's [64, V] bf16 logits all-gathered on a side stream.  Times are device times, max over ranks."""
    import torch.distributed as dist
    from matmulfreellm_b200.engine import GreedyDecoder
    from matmulfreellm_b200.models import HGRNBitConfig, HGRNBitForCausalLM
    from matmulfreellm_b200.sharding import generate_sharded
    out = {}
    # (a) correctness of the sharded path on the ranks of this run
    torch.manual_seed(0)                                   # same weights on every rank
    cfg = HGRNBitConfig(vocab_size=32000, hidden_size=256, num_hidden_layers=2, intermediate_size=704)
    tiny = HGRNBitForCausalLM(cfg).eval().to(device)
    tiny.pack_weights()
    tiny = tiny.bfloat16()
    Bt = 2 * world + 1                                     # ragged: one rank gets an extra sequence
    ids = torch.randint(0, 32000, (Bt, 12), generator=torch.Generator().manual_seed(1)).to(device)
    sharded = generate_sharded(tiny, ids, 16)
    alone = tiny.generate(ids, max_new_tokens=16)
    ok = torch.tensor([int(torch.equal(sharded, alone))], device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    out["sharded_generate_ok"] = bool(ok.item())
    del tiny

    # (b) 2.7B shapes, 64 sequences per GPU
    spec = dict(vocab_size=32000, hidden_size=2560, num_hidden_layers=32, intermediate_size=6912)
    big = build_model(args, device, spec=spec)
    Bq, steps = 64, args.throughput_steps
    dec = GreedyDecoder(big, Bq)
    dec.prefill(torch.randint(0, 32000, (Bq, 16), generator=gen).to(device))
    for _ in range(3):
        dec.step()
    main = torch.cuda.current_stream()
    side = torch.cuda.Stream(device=device)
    tok_stage = torch.empty(steps, Bq, dtype=torch.int64, device=device)
    tok_all = torch.empty(steps, world * Bq, dtype=torch.int64, device=device)
    V = spec["vocab_size"]
    logit_stage = torch.empty(2, Bq, V, dtype=torch.bfloat16, device=device)
    logit_all = torch.empty(2, world * Bq, V, dtype=torch.bfloat16, device=device)

    def run(mode):
        ev = [torch.cuda.Event() for _ in range(steps)] if mode else []
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(main)
        for t in range(steps):
            dec.step()
            if mode == "tokens":
                tok_stage[t].copy_(dec.next)             # the next step overwrites dec.next
                ev[t].record(main)
                with torch.cuda.stream(side):
                    side.wait_event(ev[t])
                    dist.all_gather_into_tensor(tok_all[t], tok_stage[t])
            elif mode == "logits":
                if t >= 2:
                    main.wait_event(done[t & 1])         # the staging slot is free once its gather has finished
                logit_stage[t & 1].copy_(dec.last_logits)
                ev[t].record(main)
                with torch.cuda.stream(side):
                    side.wait_event(ev[t])
                    dist.all_gather_into_tensor(logit_all[t & 1], logit_stage[t & 1])
                    done[t & 1].record(side)
        main.wait_stream(side)
        e1.record(main)
        e1.synchronize()
        dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=device, dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    done = [torch.cuda.Event(), torch.cuda.Event()]
    peak, _ = peaks()
    from matmulfreellm_b200.engine import bitlinear_modules
    wbytes = sum(m.packed().packed.numel() for m in bitlinear_modules(big))
    for mode, key in ((None, "no_gather"), ("tokens", "token_gather"), ("logits", "logits_gather")):
        run(mode)                                           # warm-up (NCCL channels, allocator)
        ms = run(mode)
        out[f"hgrnbit_2.7b_batch64_per_gpu_{key}"] = {
            "ms_per_step": ms, "tokens_per_s": world * Bq / (ms * 1e-3), "steps": steps,
            "whole_step_frac_of_hbm": wbytes / (ms * 1e-3) / 1e9 / peak}
    # the gathered tokens are every rank's tokens: rank r's slice of the last step equals what rank r produced
    mine = tok_all[steps - 1, rank * Bq:(rank + 1) * Bq]
    same = torch.tensor([int(torch.equal(mine, tok_stage[steps - 1]))], device=device)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    out["token_gather_consistent"] = bool(same.item())
    out["logits_gather_bytes_per_rank_per_step"] = Bq * V * 2
    del dec, big
    torch.cuda.empty_cache()
    return out


def run_ours(args):
    import torch.distributed as dist
    from matmulfreellm_b200 import _lib
    from matmulfreellm_b200.engine import GreedyDecoder, WeightStreamProbe

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    model = build_model(args, device)
    stream = torch.cuda.current_stream()
    B = args.batch
    gen = torch.Generator().manual_seed(100 + rank)
    prompt = torch.randint(0, MODEL["vocab_size"], (B, args.prompt), generator=gen)

    dec = GreedyDecoder(model, B, use_graph=not args.eager)
    dec.prefill(prompt.to(device))
    for _ in range(max(args.warmup, 3)):
        dec.step()
    barrier()

    # ---- device-resident decode: blocks of K steps, CUDA events, max over ranks ----------------------------------
    # One block = exactly --steps steps between barriers.  A block of 20 steps lasts under 20 ms, too short for the
    # clock sampler, so the block is repeated until the timed region lasts --min-seconds; the reported step time is
    # the median block (max over ranks per block), the spread is reported beside it.
    est_ms = device_time_ms(dec.step, max(args.warmup, 3), stream)
    blocks = max(1, min(2000, int(args.min_seconds * 1e3 / max(est_ms * args.steps, 1e-3)) + 1))
    with ClockSampler(local) as clocks:
        block_ms = []
        for _ in range(blocks):
            barrier()
            block_ms.append(device_time_ms(dec.step, args.steps, stream))
            barrier()
        # ---- end to end: token ids cross PCIe both ways every step ----------------------------------------
        ids_host = torch.empty(B, 1, dtype=torch.int64).pin_memory()
        out_host = torch.empty(B, dtype=torch.int64).pin_memory()
        ids_host.copy_(dec.next.cpu()[:, None])

        def e2e_step():
            # H2D of this step's input tokens, the step, D2H of its result: one graph launch (GreedyDecoder.step_host)
            dec.step_host(ids_host, out_host)
            torch.cuda.current_stream().synchronize()
            ids_host.copy_(out_host[:, None])                # the host closes the loop

        for _ in range(3):
            e2e_step()
        e2e_blocks = []
        for _ in range(max(1, blocks // 2)):
            barrier()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                e2e_step()
            torch.cuda.synchronize()
            e2e_blocks.append((time.perf_counter() - t0) / args.steps * 1e3)
            barrier()
    t = torch.tensor(block_ms + e2e_blocks, device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    block_ms, e2e_blocks = t[:blocks].tolist(), t[blocks:].tolist()
    ms, e2e_ms = median(block_ms), median(e2e_blocks)

    # ---- roofline of the dominant kernel: the BitLinear weight stream of one step -------------------------
    probe = WeightStreamProbe(model, B, torch.bfloat16, use_graph=not args.eager)
    for _ in range(3):
        probe.run()
    torch.cuda.synchronize()
    probe_ms = device_time_ms(probe.run, 10, stream)      # 325 MB of distinct weights per pass (> L2)
    peak, peak_src = peaks()
    bytes_per_launch = probe.packed_bytes / probe.launches
    achieved = probe.packed_bytes / (probe_ms * 1e-3) / 1e9
    roofline = {
        "bound": "hbm", "kernel": "bitlinear (2-bit weight stream; %d launches per step)" % probe.launches,
        "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
        "traffic": bytes_per_launch * NCU_DRAM_BYTES_PER_WEIGHT_BYTE if B == 32 else None,
        "traffic_source": "ncu dram bytes of the gate_proj launch at batch 32 (5.883 MB for 5.767 MB of packed weights), "
                          "scaled to the average launch by weight bytes; see profiles/bitlinear_mma_M32_K2048_N11264.md",
        "peak_source": peak_src, "bytes_per_launch": bytes_per_launch, "us_per_launch": probe_ms * 1e3 / probe.launches,
        "weight_bytes_per_step": probe.packed_bytes,
        "whole_step_frac": probe.packed_bytes / (ms * 1e-3) / 1e9 / peak,
    }

    kernels_per_step, packed_mb = dec.kernels_per_step, probe.packed_bytes / 1e6
    extras = {}
    if not args.no_extras and rank == 0 and world == 1:
        for b in (1, 256):
            if b == B:
                continue
            d = GreedyDecoder(model, b)
            d.prefill(torch.randint(0, MODEL["vocab_size"], (b, 16), generator=gen).to(device))
            for _ in range(3):
                d.step()
            torch.cuda.synchronize()
            m = device_time_ms(d.step, max(8, args.steps // 4), stream)
            extras[f"decode_batch{b}_tokens_per_s"] = b / (m * 1e-3)
            extras[f"decode_batch{b}_ms_per_step"] = m
            del d
        # prefill: 16 x 2048 tokens through the whole model (last-position logits only)
        pf = torch.randint(0, MODEL["vocab_size"], (16, 2048), generator=gen).to(device)
        with torch.no_grad():
            model(input_ids=pf, use_cache=True, last_token_only=True)
            torch.cuda.synchronize()
            m = device_time_ms(lambda: model(input_ids=pf, use_cache=True, last_token_only=True), 2, stream)
        extras["prefill_16x2048_tokens_per_s"] = pf.numel() / (m * 1e-3)
        extras["prefill_16x2048_ms"] = m
        del pf
        # int8 tensor-pipe peak of this GPU (bare tcgen05.mma kind::i8 loop) and the prefill BitLinear op against it
        from matmulfreellm_b200 import kernels as K
        # bare tcgen05.mma issue loop, pseudo-random operands: a 7 ms burst at the maximum clock (the 3 s loop under the
        # power cap runs at the end of the extras)
        peak_tops = K.int8_mma_peak_tops(256, 200000)
        extras["int8_tensor_peak_tops_measured"] = peak_tops
        ops = {}
        for (Kd, N) in ((2048, 2048), (2048, 11264), (5632, 2048), (2560, 2560)):
            Mtok = 16384
            w = torch.randn(N, Kd, device=device) * 0.02
            pw = K.pack_weight(w)
            del w
            q, dq, rs = K.act_quant(torch.randn(Mtok, Kd, device=device).bfloat16(), None, 1e-6)
            out = torch.empty(Mtok, N, device=device, dtype=torch.bfloat16)
            for _ in range(3):      # warm-up: steady state (the timed launches then queue behind one another)
                K.bitlinear(q, dq, rs, pw, torch.bfloat16, out=out)
            torch.cuda.synchronize()
            t = device_time_ms(lambda: K.bitlinear(q, dq, rs, pw, torch.bfloat16, out=out), 20, stream)
            tops = 2.0 * Mtok * Kd * N / (t * 1e-3) / 1e12
            ops[f"M16384_K{Kd}_N{N}"] = {"us": t * 1e3, "tops": tops, "frac_of_int8_peak": tops / peak_tops}
            del pw, q, dq, rs, out
        extras["prefill_bitlinear"] = ops
        # HGRN recurrence op (B=8, D=2048, bf16 x/o, fp32 log gate): 8 algorithmic bytes per element
        hg = {}
        peak_gbs, _ = peaks()
        for T in (2048, 8192):
            x = torch.randn(8, T, 2048, device=device).bfloat16()
            g = torch.nn.functional.logsigmoid(torch.randn(8, T, 2048, device=device))
            for _ in range(3):
                K.hgrn_scan(x, g, None, True, gate_is_log=True, state_dtype=torch.float32)
            torch.cuda.synchronize()
            t = device_time_ms(lambda: K.hgrn_scan(x, g, None, True, gate_is_log=True, state_dtype=torch.float32), 20, stream)
            gbs = 8.0 * x.numel() / (t * 1e-3) / 1e9
            hg[f"B8_T{T}_D2048"] = {"us": t * 1e3, "gb_per_s": gbs, "frac_of_hbm_peak": gbs / peak_gbs}
            del x, g
        # the scan as the model runs it on a prompt: raw i / f projections of 16 x 2048 tokens (column slabs of one
        # [B, T, 3D] bf16 tensor), gate math fused in, 6 algorithmic bytes per element
        ifg = torch.randn(16, 2048, 3 * 2048, device=device).bfloat16()
        lb = torch.rand(2048, device=device).bfloat16()
        st0 = torch.zeros(16, 2048, device=device)
        o_raw = torch.empty(16, 2048, 2048, device=device, dtype=torch.bfloat16)
        raw = lambda: K.hgrn_gated(ifg[..., :2048], ifg[..., 2048:4096], lb, st0, out=o_raw)
        for _ in range(3):
            raw()
        torch.cuda.synchronize()
        t = device_time_ms(raw, 20, stream)
        gbs = 6.0 * o_raw.numel() / (t * 1e-3) / 1e9
        hg["raw_gate_B16_T2048_D2048"] = {"us": t * 1e3, "gb_per_s": gbs, "frac_of_hbm_peak": gbs / peak_gbs}
        del ifg, lb, st0, o_raw
        extras["hgrn_scan"] = hg
        # the 2.7B shapes (32 blocks, hidden 2560, intermediate 6912) at the per-GPU batch of the 8-GPU throughput
        # configuration (512 sequences / 8)
        del dec, probe, model
        torch.cuda.empty_cache()
        big = build_model(args, device, spec=dict(vocab_size=32000, hidden_size=2560, num_hidden_layers=32, intermediate_size=6912))
        d = GreedyDecoder(big, 64)
        d.prefill(torch.randint(0, MODEL["vocab_size"], (64, 16), generator=gen).to(device))
        for _ in range(3):
            d.step()
        torch.cuda.synchronize()
        m = device_time_ms(d.step, 16, stream)
        extras["hgrnbit_2.7b_decode_batch64_tokens_per_s"] = 64 / (m * 1e-3)
        extras["hgrnbit_2.7b_decode_batch64_ms_per_step"] = m
        del d, big
        # last, because three seconds at the power cap leave the GPU at reduced clocks for what follows
        extras["int8_tensor_peak_tops_sustained"] = K.int8_mma_peak_tops(256, 24000000)

    if world > 1 and not args.no_extras:
        del dec, probe, model
        torch.cuda.empty_cache()
        extras.update(multi_gpu_extras(args, device, rank, world, gen))

    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        full_step, threads, sample, kind = cpu_reference_step_time(B, steps=3, warmup=1, budget_s=25.0)
        cpu = {"value": B / full_step, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample}

    if rank == 0:
        line = {
            "metric": METRIC, "value": world * B / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 x ternary -> int32 (bf16 activations)",
            "data": "synthetic",
            "config": config_dict(args, world),
            "timed_blocks": {"blocks_of_steps": blocks, "ms_per_step_median": ms, "ms_per_step_min": min(block_ms),
                             "ms_per_step_max": max(block_ms), "timed_region_s": sum(block_ms) * args.steps * 1e-3},
            "e2e": {"value": world * B / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8},
            "gpu_launches": kernels_per_step * args.steps * blocks,
            "weight_mb_per_step": packed_mb,
            "kernels_per_step": kernels_per_step,
            "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks.summary(), "extras": extras,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
