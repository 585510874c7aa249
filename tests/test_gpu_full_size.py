"""Parity at the full benchmark sizes (run with `-m gpu` on a B200).

Every shape whose throughput the bench quotes is compared with the CPU oracle here:
  * the BitLinear sweep at 4096 and 16384 token rows for all four layer shapes — activation codes of every row,
    int32 accumulators of 256 sampled rows, an int64 column checksum over all rows, and the bf16 output;
  * the HGRN recurrence at B = 8, D = 2048, T = 2048 and 8192 in both gate conventions;
  * a model with the 1.3B layer shapes (hidden 2048, intermediate 5632, vocabulary 32000; two blocks) in bf16:
    logits and states of a prompt pass, then 64 greedy steps at batch 32 through the CUDA-graph decoder."""
import numpy as np
import pytest
import torch

from oracle import mmfree_oracle as O

pytestmark = pytest.mark.gpu

SHAPES = [(2048, 2048), (2048, 11264), (5632, 2048), (2560, 2560)]


@pytest.fixture(scope="module")
def K():
    from matmulfreellm_b200 import _lib, kernels
    assert _lib.LIB_PATH.exists(), "libmmfree_b200.so has not been built"
    assert torch.cuda.is_available()
    return kernels


def _sample_rows(M: int, tile: int, seed: int) -> np.ndarray:
    """256 row indices: first and last rows, both sides of every kind of token-tile edge the kernels use
    (128-, 192- and 256-row tiles), and random rows."""
    rows = {0, 1, M - 1, M - 2}
    for t in (128, 192, 256):
        for e in (t, 2 * t, (M // t) * t, (M // (2 * t)) * t):
            rows.update(r for r in (e - 1, e, e + 1) if 0 <= r < M)
    rng = np.random.default_rng(seed)
    while len(rows) < 256:
        rows.add(int(rng.integers(0, M)))
    return np.array(sorted(rows)[:256])


@pytest.mark.parametrize("Kdim,N", SHAPES)
@pytest.mark.parametrize("M", [4096, 16384])
def test_bitlinear_sweep_large_m_vs_oracle(K, M, Kdim, N):
    """bf16 activations N(0,1) with 1% outlier channels x20, weights 0.02*N(0,1) ternarised: int8 codes of every row,
    int32 accumulators (256 sampled rows bit-equal, int64 column sums over all rows), fp32 output of the sampled rows
    bit-equal, and the bf16 output equal to the rounded fp32 one."""
    x, w, _ = O.bitlinear_case(M, Kdim, N, seed=M + Kdim + N)
    codes, mean = O.ternary_codes(w)
    q_ref, dq_ref, rs_ref = O.act_codes(x, None, 1e-6)
    pw = K.pack_weight(w.cuda())
    q, dq, rs = K.act_quant(x.cuda(), None, 1e-6)
    assert np.array_equal(q.cpu().numpy(), q_ref), "int8 activation codes differ"
    assert np.array_equal(dq.cpu().numpy(), dq_ref) and np.array_equal(rs.cpu().numpy(), rs_ref)
    out, acc = K.bitlinear(q, dq, rs, pw, torch.float32, return_acc=True)
    K.check_status()
    rows = _sample_rows(M, 128, seed=N)
    acc_ref = O.bitlinear_acc(q_ref[rows], codes)
    assert np.array_equal(acc[torch.from_numpy(rows).cuda()].cpu().numpy(), acc_ref), "int32 accumulators differ"
    out_ref = acc_ref.astype(np.float32) * (dq_ref[rows] * np.float32(mean))[:, None]
    assert np.array_equal(out[torch.from_numpy(rows).cuda()].cpu().numpy(), out_ref), "dequantised fp32 output differs"
    # column checksum over ALL rows: sum_m acc[m, n] == codes[n, :] . (sum_m q[m, :]), in int64
    colsum = q_ref.astype(np.int64).sum(0)
    assert np.array_equal(acc.sum(0, dtype=torch.int64).cpu().numpy(), codes.astype(np.int64) @ colsum)
    out_b = K.bitlinear(q, dq, rs, pw, torch.bfloat16)
    assert torch.equal(out_b, out.to(torch.bfloat16)), "bf16 output is not the rounded fp32 output"
    K.check_status()


def test_bitlinear_grouped_large_m(K):
    """The three-projection call of a prompt pass (i / f / g: one activation row, three code groups, three stacked weight
    matrices) at 4096 token rows equals three single-projection calls, which the sweep above compares with the oracle."""
    M, Kdim, N = 4096, 2048, 2048
    x, _, _ = O.bitlinear_case(M, Kdim, N, seed=31)
    g = torch.Generator().manual_seed(32)
    ws = [torch.randn(N, Kdim, generator=g) * 0.02 for _ in range(3)]
    nws = [1.0 + 0.1 * torch.randn(Kdim, generator=g) for _ in range(3)]
    pws = [K.pack_weight(w.cuda()) for w in ws]
    pw = K.stack_packed(pws)
    qs = [K.act_quant(x.cuda(), nw.cuda(), 1e-6) for nw in nws]
    q = torch.cat([t[0] for t in qs]); dq = torch.cat([t[1] for t in qs]); rs = torch.cat([t[2] for t in qs])
    for dt in (torch.bfloat16, torch.float32):
        out = K.bitlinear(q, dq, rs, pw, dt)
        K.check_status()
        for gi in range(3):
            single = K.bitlinear(qs[gi][0], qs[gi][1], qs[gi][2], pws[gi], dt)
            assert torch.equal(out[:, gi * N:(gi + 1) * N], single), (dt, gi)
    codes, mean = O.ternary_codes(ws[1])
    ref = O.bitlinear_int(x[:64], nws[1], codes, mean, 1e-6)[0]
    assert torch.equal(K.bitlinear(q, dq, rs, pw, torch.float32)[:64, N:2 * N].cpu(), ref)


@pytest.mark.parametrize("Kdim,N", [(2048, 2048), (2560, 2560), (5632, 2048)])
def test_bitlinear_large_m_repeatable(K, Kdim, N):
    """The same 16384-row call 60 times: every run returns the bits of the first one, whose sampled rows equal the
    oracle's.  (A synchronisation slip between the weight stream and the unpack warps once showed up as 4 - 32 wrong rows
    in one run out of seven, only with the fast bf16 epilogue; a single comparison would have missed it.)"""
    M = 16384
    x, w, _ = O.bitlinear_case(M, Kdim, N, seed=7 + Kdim)
    codes, mean = O.ternary_codes(w)
    q_ref, dq_ref, _ = O.act_codes(x, None, 1e-6)
    pw = K.pack_weight(w.cuda())
    q, dq, rs = K.act_quant(x.cuda(), None, 1e-6)
    first = K.bitlinear(q, dq, rs, pw, torch.bfloat16).clone()
    rows = _sample_rows(M, 128, seed=N)[::8]
    acc_ref = O.bitlinear_acc(q_ref[rows], codes)
    want = torch.from_numpy(acc_ref.astype(np.float32) * (dq_ref[rows] * np.float32(mean))[:, None]).to(torch.bfloat16)
    assert torch.equal(first[torch.from_numpy(rows).cuda()].cpu(), want)
    out = torch.empty_like(first)
    for rep in range(60):
        K.bitlinear(q, dq, rs, pw, torch.bfloat16, out=out)
        assert torch.equal(out, first), rep
    K.check_status()


@pytest.mark.parametrize("T", [2048, 8192])
@pytest.mark.parametrize("log", [True, False])
def test_hgrn_full_size_vs_oracle(K, T, log):
    """B = 8, D = 2048, bf16 inputs, fp32 log-forget gate (chunk_hgrn convention) or its exponential
    (fused_recurrent_hgrn convention), zero initial state: outputs rel 1e-2, fp32 final state rel 1e-4, against the
    CPU restatement of naive_recurrent_hgrn."""
    x, g_log = O.hgrn_case(8, T, 2048, seed=T, dtype=torch.bfloat16)
    g = g_log if log else torch.exp(g_log)
    o_ref, ht_ref = (O.chunk_hgrn_ref if log else O.naive_recurrent_hgrn)(x, g, None, True)
    o, ht = K.hgrn_scan(x.cuda(), g.cuda(), None, True, gate_is_log=log, state_dtype=torch.float32)
    K.check_status()
    so = o_ref.float().abs().max().item()
    assert (o.cpu().float() - o_ref.float()).abs().max().item() <= 1e-2 * so
    assert (ht.cpu() - ht_ref).abs().max().item() <= 1e-4 * ht_ref.abs().max().item()


def test_hgrn_decode_shape_vs_oracle(K):
    """Single-step update with B = 256, T = 1: the state is advanced in place."""
    g = torch.Generator().manual_seed(4)
    st = torch.randn(256, 1, 2048, generator=g)
    x1 = torch.randn(256, 1, 1, 2048, generator=g).bfloat16()
    g1 = torch.rand(256, 1, 1, 2048, generator=g)
    o_ref, ht_ref = O.naive_recurrent_hgrn(x1, g1, st, True)
    sd = st.cuda().view(256, 2048).clone()
    o1, st2 = K.hgrn_scan(x1.cuda().view(256, 1, 2048), g1.cuda().view(256, 1, 2048), sd, True, gate_is_log=False,
                          state_dtype=torch.float32, final_state_out=sd)
    assert st2.data_ptr() == sd.data_ptr()
    assert (sd.cpu() - ht_ref.view(256, 2048)).abs().max().item() <= 1e-4 * ht_ref.abs().max().item()
    assert (o1.cpu().float().view(-1) - o_ref.float().view(-1)).abs().max().item() <= 1e-2 * o_ref.float().abs().max().item()


# ----------------------------------------------------------------------------------------------------------
# model with the 1.3B layer shapes
# ----------------------------------------------------------------------------------------------------------
def _build(sd, cfg, dtype):
    import matmulfreellm_b200 as pkg
    pkg.install_as_mmfreelm()
    from mmfreelm.models import HGRNBitConfig, HGRNBitForCausalLM
    hf = HGRNBitConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, num_hidden_layers=cfg.num_hidden_layers,
                       intermediate_size=cfg.intermediate_size, rms_norm_eps=cfg.rms_norm_eps)
    model = HGRNBitForCausalLM(hf).eval()
    model.load_state_dict(sd, strict=True)
    model = model.cuda()
    model.pack_weights()
    return model.to(dtype)


def test_model_with_1p3b_layer_shapes_vs_oracle(K):
    """Hidden 2048, intermediate 5632, vocabulary 32000, two blocks, bf16 activations, weights N(0, 0.02).
    (a) prompt pass, batch 4 x 48 tokens: last-position logits and per-block states against the integer oracle;
    (b) 64 greedy steps at batch 32 through the CUDA-graph decoder (oracle.greedy_parity): a sequence may leave the
        oracle's path only at a step whose top-2 margin is within twice the logit error measured for that row in the
        teacher-forced pass of the same run; that error is bounded and the identical-token fraction is asserted."""
    from matmulfreellm_b200.engine import GreedyDecoder
    cfg = O.OracleConfig(vocab_size=32000, hidden_size=2048, num_hidden_layers=2, intermediate_size=5632)
    sd = O.random_weights(cfg, seed=13)
    model = _build(sd, cfg, torch.bfloat16)
    oracle = O.OracleHGRNBit(cfg, sd, dtype=torch.bfloat16, linear="int", bitlinear_eps=1e-6)

    ids = torch.randint(0, 32000, (4, 48), generator=torch.Generator().manual_seed(14))
    ref_logits, ref_states = oracle.forward(ids, last_only=True)
    out = model(ids.cuda(), use_cache=True, last_token_only=True)
    scale = ref_logits.float().abs().max().item()
    d = (out.logits.float().cpu() - ref_logits.float()).abs()
    # bf16 logits: one bf16 rounding step is 2^-8 relative; code flips upstream move single entries further
    assert d.median().item() <= 1e-2 * scale and d.max().item() <= 1e-1 * scale, (d.median().item() / scale, d.max().item() / scale)
    for s, r in zip(out.past_key_values, ref_states):
        ds = (s[0].float().cpu() - r).abs()
        assert ds.median().item() <= 1e-2 * r.abs().max().item() and ds.max().item() <= 1e-1 * r.abs().max().item()

    ids32 = torch.randint(0, 32000, (32, 16), generator=torch.Generator().manual_seed(15))
    dec = GreedyDecoder(model, 32)
    r = O.greedy_parity(oracle, ids32, 64, dec,
                        lambda ids: model(ids.cuda(), use_cache=False, last_token_only=True).logits[:, -1])
    assert dec.graph is not None, "the decode steps did not run from the CUDA graph"
    K.check_status()
    print(f"[1.3B shapes, batch 32, 64 steps] identical tokens {r['identical_fraction']:.4f}, {r['identical_sequences']}/32 sequences "
          f"identical over all steps; teacher-forced logit error per row: median {r['err_median']:.3e}, max {r['err_max']:.3e} "
          f"(logit scale {scale:.3f}), {r['exact_rows']:.3f} of the rows bit-identical; smallest oracle top-2 margin "
          f"{r['min_margin']:.3e}")
    # a sequence may leave the oracle's path only at a step where the oracle's top-2 margin is within twice the logit
    # error measured for that very row in the teacher-forced pass of this run
    assert r["explained"], r["violations"]
    # bf16 logits: a row differs from the oracle's by at most a few bf16 steps (2^-8 relative) ...
    assert r["err_median"] <= 2 ** -6 * scale and r["err_max"] <= 1e-1 * scale
    # ... and most tokens are the oracle's even though near-flat random-init logits tie often (measured 0.69 - 0.92:
    # the figure moves with every change of a last-bit rounding upstream, because a sequence that leaves the oracle's path
    # at an early tie differs from then on)
    assert r["identical_fraction"] >= 0.5
