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

`--impl reference` times the reference algorithm's CPU path (BitLinear.forward with per-call weight_quant,
naive_recurrent_hgrn, torch RMSNorm — restated in oracle/mmfree_oracle.py because the reference checkout
is not present on the benchmark machine) on the host cores, on a bounded sample of the same workload.
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
    return ap.parse_args()


def workload_name(args):
    return (f"HGRNBit-1.3B random-init ternarised, greedy decode, batch {args.batch} per GPU, "
            f"state seeded by a {args.prompt}-token prompt")


# dram__bytes_read+write of one bitlinear_mma_kernel launch (M=32, K=2048, N=11264) from the profiler, per byte of
# packed weights that launch streams; DRAM traffic of this kernel is the weight stream plus the activation codes
NCU_DRAM_BYTES_PER_WEIGHT_BYTE = 6.124 / 5.767


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
def cpu_reference_step_time(batch: int, steps: int, warmup: int, budget_s: float):
    """Time one decode step of the reference's CPU path.  A full 1.3B step on CPU re-ternarises every weight
    (as the reference does on each call), so the sample is the first `n_layers` of the 24 layers plus the
    lm_head, and the step time is extrapolated linearly in the layer count; n_layers is chosen from a
    one-layer calibration so that warmup + steps fit in `budget_s`."""
    from oracle import mmfree_oracle as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    cfg1 = O.OracleConfig(**{**MODEL, "num_hidden_layers": 1})
    ids = torch.randint(0, MODEL["vocab_size"], (batch, 1), generator=torch.Generator().manual_seed(0))

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

    m1 = build(1)
    timed(m1, 1)
    t1 = min(timed(m1, 2))                       # one layer + lm_head
    # head-only estimate: a 0-layer model is just final norm + lm_head
    m0 = build(0)
    timed(m0, 1)
    t_head = min(timed(m0, 2))
    t_layer = max(t1 - t_head, 1e-4)
    total_steps = steps + warmup
    n_layers = int(max(1, min(MODEL["num_hidden_layers"], (budget_s / total_steps - t_head) / t_layer)))
    model = m1 if n_layers == 1 else build(n_layers)
    timed(model, warmup)
    ts = timed(model, steps)
    mean = sum(ts) / len(ts)
    per_layer = (mean - t_head) / n_layers
    full_step = t_head + per_layer * MODEL["num_hidden_layers"]
    sample = (f"batch {batch}, 1 new token, first {n_layers} of {MODEL['num_hidden_layers']} layers + lm_head in "
              f"fp32 (weight_quant re-evaluated per call as in the reference), {steps} steps; full-step time "
              f"extrapolated linearly in the layer count")
    return full_step, threads, sample


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    full_step, threads, sample = cpu_reference_step_time(args.batch, args.steps, args.warmup, budget_s=150.0)
    value = args.batch / full_step
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": full_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "device": "host CPU"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
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

    # ---- device-resident decode: K steps, CUDA events, max over ranks -------------------------------------
    with ClockSampler(local) as clocks:
        barrier()
        ms = device_time_ms(dec.step, args.steps, stream)
        barrier()
        # keep the sampler running over the end-to-end loop too
        # ---- end to end: token ids cross PCIe both ways every step ----------------------------------------
        ids_host = torch.empty(B, 1, dtype=torch.int64).pin_memory()
        out_host = torch.empty(B, dtype=torch.int64).pin_memory()
        ids_host.copy_(dec.next.cpu()[:, None])

        def e2e_step():
            dec.ids.copy_(ids_host, non_blocking=True)       # H2D: this step's input tokens
            dec.step()
            out_host.copy_(dec.next, non_blocking=True)      # D2H: the step's result
            torch.cuda.current_stream().synchronize()
            ids_host.copy_(out_host[:, None])                # the host closes the loop

        for _ in range(3):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        torch.cuda.synchronize()
        e2e_s = (time.perf_counter() - t0) / args.steps
        barrier()
    t = torch.tensor([ms, e2e_s * 1e3], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()

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
        "traffic_source": "ncu dram bytes of the gate_proj launch at batch 32 (6.124 MB for 5.767 MB of packed weights), "
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
            K.bitlinear(q, dq, rs, pw, torch.bfloat16, out=out)
            torch.cuda.synchronize()
            t = device_time_ms(lambda: K.bitlinear(q, dq, rs, pw, torch.bfloat16, out=out), 5, stream)
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
            K.hgrn_scan(x, g, None, True, gate_is_log=True, state_dtype=torch.float32)
            torch.cuda.synchronize()
            t = device_time_ms(lambda: K.hgrn_scan(x, g, None, True, gate_is_log=True, state_dtype=torch.float32), 5, stream)
            gbs = 8.0 * x.numel() / (t * 1e-3) / 1e9
            hg[f"B8_T{T}_D2048"] = {"us": t * 1e3, "gb_per_s": gbs, "frac_of_hbm_peak": gbs / peak_gbs}
            del x, g
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

    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        full_step, threads, sample = cpu_reference_step_time(B, steps=2, warmup=1, budget_s=25.0)
        cpu = {"value": B / full_step, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}

    if rank == 0:
        line = {
            "metric": METRIC, "value": world * B / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 x ternary -> int32 (bf16 activations)",
            "data": "synthetic",
            "config": {"workload": workload_name(args), "per_gpu_batch": B, "global_batch": world * B,
                       "parallelism": f"batch-sharded x{world}, no data-path collective",
                       "l2_policy": "inputs larger than L2: one step streams %.0f MB of packed weights (L2 = 126 MB)"
                                    % packed_mb},
            "e2e": {"value": world * B / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8},
            "gpu_launches": kernels_per_step * args.steps,
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
