"""Op-level micro-benchmarks of the C-ABI kernels (also the command lines used for profiler captures).

    python -m matmulfreellm_b200.opbench bitlinear --M 32 --K 2048 --N 11264 [--kernel auto|gemv|mma|decode] [--iters 20]
    python -m matmulfreellm_b200.opbench hgrn --B 8 --T 2048 --D 2048 [--gate log|linear]
    python -m matmulfreellm_b200.opbench rowwise --M 4096 --D 2048
    python -m matmulfreellm_b200.opbench int8peak
    python -m matmulfreellm_b200.opbench sync           (grid-wide barrier and CTA-to-CTA signal cost)
    python -m matmulfreellm_b200.opbench chain --M 32   (the BitLinear launches of one decode step as a dependent chain)
    python -m matmulfreellm_b200.opbench timeline --batch 32   (experiments build: where a decode step's kernels spend time)
    python -m matmulfreellm_b200.opbench prefill --batch 16 --seq 2048 --layers 2
    python -m matmulfreellm_b200.opbench sweep          (the BitLinear op sweep: 5 token counts x 4 layer shapes)

Each prints one JSON line: device time per call (CUDA events, after 3 warm-ups) and the achieved GB/s of
algorithmic bytes and/or TOP/s.  Inputs are seeded synthetic data; every repetition of `bitlinear` uses a
different weight buffer (round-robin over --buffers) so that small layers are streamed from HBM, not from L2.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import kernels as K


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


def bitlinear(a):
    if a.kernel == "decode":      # the mma.sync decode experiment exists in the experiments build only
        from . import _lib
        with _lib.experiments_library():
            return _bitlinear(a)
    return _bitlinear(a)


def _bitlinear(a):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    nbuf = max(1, a.buffers)
    pws = []
    for _ in range(nbuf):
        w = torch.randn(a.N, a.K, device=dev, generator=g) * 0.02
        pws.append(K.pack_weight(w))
        del w
    x = torch.randn(a.M, a.K, device=dev, generator=g)
    x[:, torch.randperm(a.K, device=dev, generator=g)[: a.K // 100]] *= 20
    q, dq, rs = K.act_quant(x.bfloat16(), None, 1e-6)
    out = torch.empty(a.M, a.N, device=dev, dtype=torch.bfloat16)
    kern = {"auto": K.KERNEL_AUTO, "gemv": K.KERNEL_GEMV, "mma": K.KERNEL_MMA, "decode": K.KERNEL_STREAM}[a.kernel]
    state = {"i": 0}

    def fn():
        K.bitlinear(q, dq, rs, pws[state["i"] % nbuf], torch.bfloat16, kernel=kern, out=out)
        state["i"] += 1

    graph = None
    if a.graph:      # replay `--graph` back-to-back launches from one CUDA graph (device time without host launch cost)
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(a.graph):
                fn()
        t = _time(graph.replay, a.iters) / a.graph
    else:
        t = _time(fn, a.iters)
    wbytes = a.K * a.N / 4
    print(json.dumps({"op": "bitlinear", "M": a.M, "K": a.K, "N": a.N, "kernel": a.kernel, "us": t * 1e6,
                      "weight_stream_gb_per_s": wbytes / t / 1e9, "tops": 2.0 * a.M * a.K * a.N / t / 1e12,
                      "algorithmic_bytes": wbytes + a.M * a.K + 2 * a.M * a.N}))


def hgrn(a):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    glog = torch.nn.functional.logsigmoid(torch.randn(a.B, a.T, a.D, device=dev, generator=g))
    x = ((1 - glog.exp()) * torch.nn.functional.silu(torch.randn(a.B, a.T, a.D, device=dev, generator=g))).bfloat16()
    gate = glog if a.gate == "log" else glog.exp()
    h0 = torch.zeros(a.B, a.D, device=dev)
    fn = lambda: K.hgrn_scan(x, gate, h0, True, gate_is_log=a.gate == "log", state_dtype=torch.float32)
    per_element = 8.0
    if a.gate == "raw":     # the in-model op: raw i / f projection outputs (slabs of one [B,T,3D] tensor), gate math fused in
        ifg = torch.randn(a.B, a.T, 3 * a.D, device=dev, generator=g).bfloat16()
        lb = torch.rand(a.D, device=dev, generator=g).bfloat16()
        o = torch.empty(a.B, a.T, a.D, device=dev, dtype=torch.bfloat16)
        fn = lambda: K.hgrn_gated(ifg[..., :a.D], ifg[..., a.D:2 * a.D], lb, h0, out=o)
        per_element = 6.0
    if getattr(a, "graph", 0):     # small problems: device time without host launch cost
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(a.graph):
                fn()
        t = _time(graph.replay, a.iters) / a.graph
    else:
        t = _time(fn, a.iters)
    nbytes = per_element * x.numel() + (8.0 * a.B * a.D if a.T == 1 else 0.0)     # a single step also reads and writes the state
    print(json.dumps({"op": "hgrn_scan", "gate": a.gate, "B": a.B, "T": a.T, "D": a.D, "us": t * 1e6, "algorithmic_bytes": nbytes,
                      "gb_per_s": nbytes / t / 1e9}))


def rowwise(a):
    dev = torch.device("cuda")
    x = torch.randn(a.M, a.D, device=dev).bfloat16()
    res = torch.randn(a.M, a.D, device=dev).bfloat16()
    nw = torch.ones(a.D, device=dev)
    t = _time(lambda: K.prenorm_quant(x, res, nw, 1e-6, [nw, nw, nw], 1e-6, False, want_residual_out=True), a.iters)
    nbytes = a.M * a.D * (2 + 2 + 2 + 3)
    print(json.dumps({"op": "prenorm_quant(3 groups)", "M": a.M, "D": a.D, "us": t * 1e6, "algorithmic_bytes": nbytes,
                      "gb_per_s": nbytes / t / 1e9}))


def sync(a):
    barrier, signal, chain_pdl, chain_plain = K.sync_probe(2000)
    print(json.dumps({"op": "sync", "grid_barrier_us": barrier, "cta_to_cta_signal_us": signal,
                      "dependent_kernel_chain_us_per_kernel": {"programmatic_dependent_launch": chain_pdl, "plain": chain_plain},
                      "what": "one barrier among one resident CTA per SM (release add + acquire poll on one counter); one "
                              "release store -> acquire poll hand-over between two CTAs; 200 dependent trivial kernels "
                              "(one CTA per SM) replayed from a CUDA graph"}))


def _model(layers):
    from .models import HGRNBitConfig, HGRNBitForCausalLM
    from .ops.fusedbitnet import BitLinear
    dev = torch.device("cuda")
    cfg = HGRNBitConfig(vocab_size=32000, hidden_size=2048, num_hidden_layers=layers, intermediate_size=5632)
    with torch.device(dev):
        model = HGRNBitForCausalLM(cfg).eval()
    g = torch.Generator(device=dev).manual_seed(1234)
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, BitLinear):
                m.weight.normal_(0.0, 0.02, generator=g)
        model.model.embeddings.weight.normal_(0.0, 0.02, generator=g)
    model.pack_weights()
    return model.to(torch.bfloat16)


def chain(a):
    """The 97 BitLinear contractions of one HGRNBit-1.3B decode step (pre-quantised inputs, nothing else) replayed from
    a CUDA graph as a dependent chain, per kernel: the tcgen05 kernel, the dp4a GEMV, and (experiments build) the
    mma.sync decode experiment."""
    from . import _lib, engine
    model = _model(24)
    orig = K.bitlinear
    out = {"op": "chain", "M": a.M, "launches": 97}

    def run(kernel):
        def forced(q, dq, rs, pw, dt, kernel_=None, return_acc=False, out=None, **kw):
            return orig(q, dq, rs, pw, dt, kernel=kernel, return_acc=return_acc, out=out)
        K.bitlinear = forced
        try:
            probe = engine.WeightStreamProbe(model, a.M, torch.bfloat16)
            t = _time(probe.run, a.iters)
            return {"us_per_launch": t * 1e6 / probe.launches, "weight_gb_per_s": probe.packed_bytes / t / 1e9}
        finally:
            K.bitlinear = orig

    out["tcgen05"] = run(K.KERNEL_MMA)
    out["gemv_dp4a"] = run(K.KERNEL_GEMV)
    with _lib.experiments_library():
        out["mma_sync_experiment"] = run(K.KERNEL_STREAM)
    print(json.dumps(out))


def timeline(a):
    """Experiments build: global-timer stamps of CTA 0 of every prenorm_quant launch of one decode step (replayed from
    a CUDA graph): how long after the grid dependency resolves the row is loaded, reduced, normalised and quantised, and
    how far apart consecutive launches of the chain are."""
    from . import _lib
    from .engine import GreedyDecoder
    with _lib.experiments_library() as lib:
        model = _model(a.layers)
        buf = torch.zeros(8 + 8 * 1000, dtype=torch.int64, device="cuda")
        lib.mmf_row_trace(buf.data_ptr())          # before the capture: the pointer is baked into the graph
        try:
            dec = GreedyDecoder(model, a.batch)
            dec.prefill(torch.randint(0, 32000, (a.batch, 8), device="cuda"))
            for _ in range(3):
                dec.step()
            torch.cuda.synchronize()
            buf.zero_()
            torch.cuda.synchronize()
            dec.step()
            torch.cuda.synchronize()
        finally:
            lib.mmf_row_trace(None)
        # the same step with the tcgen05 kernel's trace armed (word 1 of the split-K workspace of the capture stream)
        for ws in list(K._ws_cache.values()):
            w32 = ws.view(torch.int32)
            w32[2] = 0
            w32[1] = 0x7ACE
        torch.cuda.synchronize()
        dec.step()
        torch.cuda.synchronize()
        mma_rows = []
        for ws in list(K._ws_cache.values()):
            w32 = ws.view(torch.int32)
            m = int(w32[2].item())
            w32[1] = 0
            w32[2] = 0
            if m == 0:
                continue
            r = ws[64:64 + m * 256].view(torch.int64).view(m, 32).cpu()
            for i in range(m):
                v = r[i].tolist()
                mm = [x for x in v[8:16] if x > 0]
                if not mm:
                    continue
                m0 = mm[0]
                mma_rows.append({"start_before_first_mma_ns": int(m0 - v[0]), "last_mma_issue_ns": int(mm[-1] - m0),
                                 "accumulators_complete_ns": int(v[4] - m0), "partials_pushed_ns": int(v[5] - m0),
                                 "cluster_barrier_done_ns": int(v[6] - m0) if v[6] > 0 else None, "end_ns": int(v[7] - m0),
                                 "previous_end_to_first_mma_ns": int(m0 - r[i - 1, 7]) if i else None})
        n = int(buf.view(torch.int32)[0].item())
        rec = buf[8:8 + 8 * n].view(n, 8).cpu()
        rows = []
        for i in range(n):
            r = [int(x - rec[i, 2]) for x in rec[i].tolist()]
            rows.append({"start_before_release_ns": -r[0], "row_loaded_ns": r[3], "first_sum_ns": r[4], "second_norm_ns": r[5],
                         "codes_written_ns": r[6], "end_ns": r[7],
                         "since_previous_release_ns": int(rec[i, 2] - rec[i - 1, 2]) if i else None})
        med = lambda key: sorted(x[key] for x in rows[1:])[len(rows[1:]) // 2]
        print(json.dumps({"op": "timeline", "batch": a.batch, "layers": a.layers, "prenorm_quant_launches": n,
                          "median_ns_after_release": {k: med(k) for k in ("row_loaded_ns", "first_sum_ns", "second_norm_ns",
                                                                            "codes_written_ns", "end_ns")},
                          "median_ns_between_prenorm_releases": med("since_previous_release_ns"), "first_launches": rows[:5],
                          "tcgen05_kernel_launches_ns_after_first_mma": mma_rows[:9]}))


def int8peak(a):
    """Bare tcgen05.mma kind::i8 issue loop with pseudo-random operands: a burst of about 7 ms (the GPU holds its
    maximum clock) and a loop of about 3 s (the clock settles under the power cap)."""
    print(json.dumps({"op": "int8_mma_peak", "tops_n256_burst": K.int8_mma_peak_tops(256, 200000),
                      "tops_n256_sustained": K.int8_mma_peak_tops(256, 24000000),
                      "tops_n192_burst": K.int8_mma_peak_tops(192, 200000), "tops_n128_burst": K.int8_mma_peak_tops(128, 200000),
                      "tops_n32_burst": K.int8_mma_peak_tops(32, 200000)}))


def prefill(a):
    """Prompt pass of a random-init HGRNBit with the 1.3B layer shapes (hidden 2048, intermediate 5632, vocab 32000) and
    `--layers` blocks through the fused chain; last-position logits only."""
    dev = torch.device("cuda")
    model = _model(a.layers)
    g = torch.Generator(device=dev).manual_seed(99)
    ids = torch.randint(0, 32000, (a.batch, a.seq), device=dev, generator=g)
    with torch.no_grad():
        t = _time(lambda: model(input_ids=ids, use_cache=True, last_token_only=True), a.iters)
    print(json.dumps({"op": "prefill", "batch": a.batch, "seq": a.seq, "layers": a.layers, "ms": t * 1e3,
                      "tokens_per_s_per_layer_block": a.batch * a.seq / t * a.layers}))


def pfknobs(a):
    """The persistent prefill BitLinear kernel under its experiment switches (experiments build): every compiled shape
    (`MMF_TUNE_PERSISTENT` = 10 + v) and, for the default shape, the timing-only switches that leave out the activation
    loads (1), the 2-bit expansion (2), the output stores (4) or all three (7) — results are wrong with a switch on, only
    the time means something; then the timeline of CTA 0 (global timer) for the first work items; then a bare issue
    loop with one thread, two threads and a pair of CTAs.  3 warm-up + 20 timed launches per figure; over a run this long
    the GPU settles under its power cap, so later figures read lower than the first (the traced launch reports its SM clock)."""
    from matmulfreellm_b200 import _lib
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(a.M, a.K, device=dev, generator=g).bfloat16()
    w = torch.randn(a.N, a.K, device=dev, generator=g) * 0.02
    pw = K.pack_weight(w)
    q, dq, rs = K.act_quant(x, None, 1e-6)
    out = torch.empty(a.M, a.N, device=dev, dtype=torch.bfloat16)
    fn = lambda: K.bitlinear(q, dq, rs, pw, torch.bfloat16, out=out)
    ops = 2.0 * a.M * a.K * a.N
    res = {"op": "prefill_kernel_experiments", "M": a.M, "K": a.K, "N": a.N}
    with _lib.experiments_library() as lib:
        peak = K.int8_mma_peak_tops(256, 200000)
        res["int8_peak_tops"] = peak
        shapes = {}
        for v in (0, 1, 2, 5, 6, 7, 8, 9, 10, 11):
            lib.mmf_tuning(7, 10 + v if v else 0)
            try:
                t = _time(fn, 20)
                shapes[f"shape_{v}"] = {"us": t * 1e6, "frac_of_int8_peak": ops / t / 1e12 / peak}
            except _lib.MMFreeError as e:
                shapes[f"shape_{v}"] = {"refused": str(e)[:80]}
        lib.mmf_tuning(7, 0)
        res["compiled_shapes"] = shapes
        skips = {}
        for bits in (0, 1, 2, 4, 7):
            lib.mmf_tuning(12, bits)
            t = _time(fn, 20)
            skips[f"skip_{bits}"] = {"us": t * 1e6, "frac_of_int8_peak": ops / t / 1e12 / peak}
        lib.mmf_tuning(12, 0)
        res["parts_switched_off"] = skips
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ws = list(K._ws_cache.values())[0]
        w32 = ws.view(torch.int32)
        w32[1] = 0x7ACE
        torch.cuda.synchronize()
        fn()
        torch.cuda.synchronize()
        w32[1] = 0
        rec = ws[32:32 + 28 * 8].view(torch.int64).cpu().tolist()
        ws[32:32 + 28 * 8].zero_()
        rel = [(v - rec[0]) if v else 0 for v in rec]
        res["timeline_cta0_ns"] = {
            "sm_clock_ghz": (rec[27] - rec[26]) / max(1, rec[25] - rec[0]),
            "mma_thread_items_1_to_4_start_firststage_allissued": [rel[1 + i * 3:4 + i * 3] for i in range(4)],
            "epilogue_items_0_to_3_accfull_handedback_stored": [rel[13 + i * 3:16 + i * 3] for i in range(4)]}
        loop = {}
        for commits in (0, 1):
            lib.mmf_tuning(8, commits)
            for n in (64, 128, 192):
                for mode, name in ((1, "one_thread"), (2, "two_threads"), (3, "cta_pair")):
                    if mode == 2 and n > 128:
                        continue
                    lib.mmf_tuning(11, mode)
                    loop[f"commits_per_4_mma_{commits}_columns_{n}_{name}"] = K.int8_mma_peak_tops(n, 100000)
        res["bare_issue_loop_tops"] = loop
    print(json.dumps(res))


def sweep(a):
    """FusedBitLinear op sweep: M in {1,16,256,4096,16384} x (K,N) in {(2048,2048),(2048,11264),(5632,2048),(2560,2560)}.
    Small M: 24 launches over 24 distinct weight buffers (more than L2 in total for the larger shapes) replayed from one
    CUDA graph, so the figure is device time per launch with the weights streamed from HBM; the launches in the graph
    overlap their prologues (programmatic dependent launch), as they do inside a decode step."""
    class Args:
        pass
    for (Kd, N) in ((2048, 2048), (2048, 11264), (5632, 2048), (2560, 2560)):
        for M in (1, 16, 256, 4096, 16384):
            b = Args()
            b.M, b.K, b.N, b.kernel, b.iters = M, Kd, N, "auto", 5
            b.buffers, b.graph = (24, 24) if M <= 256 else (1, 0)
            bitlinear(b)
    for (B, T) in ((8, 2048), (8, 8192), (256, 1)):
        h = Args()
        h.B, h.T, h.D, h.gate, h.iters = B, T, 2048, "log", 10
        h.graph = 20 if T == 1 else 0
        hgrn(h)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="op", required=True)
    b = sub.add_parser("bitlinear")
    b.add_argument("--M", type=int, default=32); b.add_argument("--K", type=int, default=2048)
    b.add_argument("--N", type=int, default=11264); b.add_argument("--kernel", default="auto")
    b.add_argument("--iters", type=int, default=20); b.add_argument("--buffers", type=int, default=1)
    b.add_argument("--graph", type=int, default=0)
    h = sub.add_parser("hgrn")
    h.add_argument("--B", type=int, default=8); h.add_argument("--T", type=int, default=2048)
    h.add_argument("--D", type=int, default=2048); h.add_argument("--gate", default="log"); h.add_argument("--iters", type=int, default=10)
    h.add_argument("--graph", type=int, default=0)
    r = sub.add_parser("rowwise")
    r.add_argument("--M", type=int, default=4096); r.add_argument("--D", type=int, default=2048); r.add_argument("--iters", type=int, default=10)
    sub.add_parser("int8peak")
    pk = sub.add_parser("pfknobs")
    pk.add_argument("--M", type=int, default=16384); pk.add_argument("--K", type=int, default=2048)
    pk.add_argument("--N", type=int, default=11264)
    sub.add_parser("sync")
    ch = sub.add_parser("chain")
    ch.add_argument("--M", type=int, default=32); ch.add_argument("--iters", type=int, default=20)
    tl = sub.add_parser("timeline")
    tl.add_argument("--batch", type=int, default=32); tl.add_argument("--layers", type=int, default=4)
    sub.add_parser("sweep")
    pf = sub.add_parser("prefill")
    pf.add_argument("--batch", type=int, default=16); pf.add_argument("--seq", type=int, default=2048)
    pf.add_argument("--layers", type=int, default=2); pf.add_argument("--iters", type=int, default=2)
    a = ap.parse_args()
    {"bitlinear": bitlinear, "hgrn": hgrn, "rowwise": rowwise, "int8peak": int8peak, "sync": sync, "chain": chain, "timeline": timeline, "prefill": prefill, "sweep": sweep, "pfknobs": pfknobs}[a.op](a)


if __name__ == "__main__":
    main()
