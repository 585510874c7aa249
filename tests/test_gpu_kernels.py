"""GPU parity tests of the C-ABI kernels against the CPU oracle (run with `-m gpu` on a B200).

Bit-exact: ternary codes and their packed layout, int8 activation codes, per-row scales, int32
accumulators, and the fp32 dequantised output (its two fp32 products are ordered the same on both sides).
Within tolerance: anything that passes through exp / sigmoid or a bf16 rounding (stated per test)."""
import numpy as np
import pytest
import torch

from oracle import mmfree_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from matmulfreellm_b200 import _lib, kernels
    assert _lib.LIB_PATH.exists(), "libmmfree_b200.so has not been built"
    assert torch.cuda.is_available()
    return kernels


def dev(t):
    return t.cuda()


# ----------------------------------------------------------------------------------------------------------
# offline ternarisation + packing
# ----------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("N,Kdim", [(128, 64), (128, 256), (200, 192), (384, 704), (2048, 2048), (2560, 2560)])
def test_pack_ternary_bit_exact(K, N, Kdim):
    g = torch.Generator().manual_seed(N * 7 + Kdim)
    w = torch.randn(N, Kdim, generator=g) * 0.02
    codes, mean = O.ternary_codes(w)
    pw = K.pack_weight(dev(w))
    assert pw.scale.cpu().numpy()[0] == mean
    got = pw.packed.cpu().numpy().view(np.uint32)
    assert np.array_equal(got, O.pack_ternary(codes))
    assert np.array_equal(K.unpack_codes(pw).cpu().numpy(), codes)


def test_pack_ternary_edge_values(K):
    """All-zero weights (mean clamps to 1e-5), exact ties (round half to even) and huge values (clamp to +-1)."""
    w = torch.zeros(128, 64)
    pw = K.pack_weight(dev(w))
    assert pw.scale.item() == np.float32(1e-5) and int(K.unpack_codes(pw).abs().sum()) == 0
    w = torch.full((128, 64), 1.0)
    w[0, :8] = torch.tensor([0.5, -0.5, 1.5, -1.5, 2.5, 100.0, -100.0, 0.0])
    codes, mean = O.ternary_codes(w)
    pw = K.pack_weight(dev(w))
    assert pw.scale.item() == mean
    assert np.array_equal(K.unpack_codes(pw).cpu().numpy(), codes)


def test_pack_matches_reference_weight_quant(K, golden):
    q = golden["quant_cases"]
    for idx, (M, Kd, N, seed) in enumerate(q["cases"]):
        _, w, _ = O.bitlinear_case(int(M), int(Kd), int(N), seed=int(seed), dtype=torch.float32)
        pw = K.pack_weight(dev(w))
        assert np.array_equal(K.unpack_codes(pw).cpu().numpy(), q[f"c{idx}_wq_sign"])


# ----------------------------------------------------------------------------------------------------------
# RMSNorm + activation quantisation
# ----------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("M,Kdim", [(1, 256), (7, 704), (16, 2048), (5, 5632), (3, 2560), (2, 6912)])
def test_act_quant_bit_exact(K, dtype, M, Kdim):
    x, _, _ = O.bitlinear_case(M, Kdim, 128, seed=M + Kdim, dtype=dtype)
    g = torch.Generator().manual_seed(5)
    nw = 1.0 + 0.1 * torch.randn(Kdim, generator=g)
    for eps, weight in [(1e-6, nw), (1e-8, None)]:
        q_ref, dq_ref, rs_ref = O.act_codes(x, weight, eps)
        q, dq, rs = K.act_quant(dev(x), None if weight is None else dev(weight), eps)
        assert np.array_equal(q.cpu().numpy(), q_ref)
        assert np.array_equal(dq.cpu().numpy(), dq_ref)
        assert np.array_equal(rs.cpu().numpy(), rs_ref)


def test_act_quant_edge_rows(K):
    """Zero row (absmax clamps to 1e-5), a row with one huge outlier, no-norm mode, strided input, M = 0."""
    x = torch.randn(4, 256)
    x[1] = 0
    x[2, 17] = 3e4
    for use_norm in (True, False):
        q_ref, dq_ref, rs_ref = O.act_codes(x, None, 1e-6, use_norm=use_norm)
        q, dq, rs = K.act_quant(dev(x), None, 1e-6, use_norm=use_norm)
        assert np.array_equal(q.cpu().numpy(), q_ref) and np.array_equal(dq.cpu().numpy(), dq_ref)
        assert np.array_equal(rs.cpu().numpy(), rs_ref)
    wide = dev(torch.randn(4, 512).bfloat16())
    view = wide[:, :256]                      # row stride 512
    q, dq, _ = K.act_quant(view, None, 1e-6)
    q_ref, dq_ref, _ = O.act_codes(view.cpu(), None, 1e-6)
    assert np.array_equal(q.cpu().numpy(), q_ref) and np.array_equal(dq.cpu().numpy(), dq_ref)
    q, dq, rs = K.act_quant(dev(torch.zeros(0, 256)), None, 1e-6)
    assert q.shape == (0, 256)


def test_act_quant_matches_reference_activation_quant(K, golden):
    """Against the reference's own activation_quant output: identical codes except at rounding ties that its
    fp32-accumulated row norm resolves the other way."""
    q = golden["quant_cases"]
    for idx in range(len(q["cases"])):
        x, nw, xn = torch.from_numpy(q[f"c{idx}_x"]), torch.from_numpy(q[f"c{idx}_nw"]), q[f"c{idx}_xn"]
        codes, dq, _ = K.act_quant(dev(x), dev(nw), 1e-8)
        s = np.float32(127.0) / np.maximum(np.abs(xn).max(-1, keepdims=True), np.float32(1e-5))
        ref_codes = np.rint(q[f"c{idx}_actq"] * s)
        pre = xn * s
        near_tie = np.abs(np.abs(pre - np.floor(pre)) - 0.5) < 1e-3
        diff = codes.cpu().numpy() != ref_codes
        assert np.all(~diff | near_tie) and diff.sum() <= 2


# ----------------------------------------------------------------------------------------------------------
# BitLinear contraction
# ----------------------------------------------------------------------------------------------------------
def _bitlinear_check(K, M, Kdim, N, kernel, dtype=torch.bfloat16, seed=0):
    x, w, _ = O.bitlinear_case(M, Kdim, N, seed=seed, dtype=dtype)
    codes, mean = O.ternary_codes(w)
    out_ref, acc_ref, q_ref, dq_ref = O.bitlinear_int(x, None, codes, mean, 1e-6, out_dtype=torch.float32)
    pw = K.pack_weight(dev(w))
    q, dq, rs = K.act_quant(dev(x), None, 1e-6)
    assert np.array_equal(q.cpu().numpy(), q_ref)
    out, acc = K.bitlinear(q, dq, rs, pw, torch.float32, kernel=kernel, return_acc=True)
    assert np.array_equal(acc.cpu().numpy(), acc_ref), "int32 accumulators differ"
    assert np.array_equal(out.cpu().numpy(), out_ref.numpy()), "dequantised fp32 output differs"
    # and the activation-dtype output is the correctly rounded fp32 one
    out_b = K.bitlinear(q, dq, rs, pw, dtype, kernel=kernel)
    assert torch.equal(out_b.cpu(), out_ref.to(dtype))
    # the split-K workspace must be left zeroed: a second call gives the same answer
    out2 = K.bitlinear(q, dq, rs, pw, torch.float32, kernel=kernel)
    assert torch.equal(out2, out)
    K.check_status()          # no bounded device-side wait gave up
    return out_ref


GEMV_CASES = [(1, 256, 128), (1, 2048, 2048), (2, 704, 256), (3, 2048, 384), (4, 5632, 2048), (5, 2560, 2560),
              (8, 2048, 11264), (16, 2048, 2048), (33, 704, 256), (1, 2048, 200)]


@pytest.mark.parametrize("M,Kdim,N", GEMV_CASES)
def test_bitlinear_gemv_bit_exact(K, M, Kdim, N):
    _bitlinear_check(K, M, Kdim, N, K.KERNEL_GEMV)


MMA_CASES = [(8, 256, 128), (16, 2048, 2048), (32, 2048, 11264), (64, 5632, 2048), (256, 2560, 2560),
             (5, 704, 256), (33, 2048, 384), (100, 2048, 200), (256, 2048, 2048), (1, 2048, 2048)]


@pytest.mark.parametrize("M,Kdim,N", MMA_CASES)
def test_bitlinear_mma_bit_exact(K, M, Kdim, N):
    _bitlinear_check(K, M, Kdim, N, K.KERNEL_MMA)


STREAM_CASES = [(1, 256, 128), (1, 2048, 2048), (2, 704, 256), (4, 5632, 2048), (5, 704, 256), (8, 2048, 11264),
                (16, 2048, 2048), (24, 2560, 2560), (32, 2048, 11264), (32, 5632, 2048), (33, 2048, 384), (64, 2560, 2560),
                (64, 2048, 200), (17, 2048, 200), (3, 6912, 2560), (32, 6912, 2560), (64, 5632, 2048), (40, 2048, 32000)]


@pytest.mark.parametrize("M,Kdim,N", STREAM_CASES)
def test_bitlinear_stream_bit_exact(K, M, Kdim, N):
    """The mma.sync decode experiment (persistent CTAs, resident codes, 16 rows x 8 tokens per MMA; experiments build
    only): every token-tile count 1..8, a ragged last slab (N = 200), K with a trailing chunk group (704 = 11 chunks),
    and problems whose codes do not fit in shared memory at once (32 x 6912, 64 x 5632: two launches over token blocks)."""
    from matmulfreellm_b200 import _lib
    with _lib.experiments_library():
        _bitlinear_check(K, M, Kdim, N, K.KERNEL_STREAM)


def test_bitlinear_stream_layout_and_strided_output(K):
    """Slab-major copy of the packed codes, and strided output rows (ld_out > N), in the experiments build."""
    from matmulfreellm_b200 import _lib
    x, w, _ = O.bitlinear_case(32, 2048, 384, seed=5)
    pw = K.pack_weight(dev(w))
    q, dq, rs = K.act_quant(dev(x), None, 1e-6)
    a, acc_a = K.bitlinear(q, dq, rs, pw, torch.bfloat16, return_acc=True)
    with _lib.experiments_library():
        b, acc_b = K.bitlinear(q, dq, rs, pw, torch.bfloat16, kernel=K.KERNEL_STREAM, return_acc=True)
        wide = torch.zeros(32, 512, dtype=torch.bfloat16, device="cuda")
        K.bitlinear(q, dq, rs, pw, torch.bfloat16, kernel=K.KERNEL_STREAM, out=wide[:, 64:448])
    assert torch.equal(a, b) and torch.equal(acc_a, acc_b)
    assert torch.equal(wide[:, 64:448], a) and int(wide[:, :64].abs().sum()) == 0 and int(wide[:, 448:].abs().sum()) == 0
    # the same 16-byte pieces, slab-major ([tile][slab of 16 rows][chunk][row][16 B])
    got = pw.packed.cpu().numpy().view(np.uint32)
    want = got.reshape(3, 32, 8, 16, 4).transpose(0, 2, 1, 3, 4).reshape(-1)
    assert np.array_equal(pw.slabs.cpu().numpy().view(np.uint32), want)
    K.check_status()


@pytest.mark.parametrize("M", [1, 4, 32])
def test_bitlinear_grouped(K, M):
    """Three projections sharing an input row but not a norm weight, run as one grouped launch."""
    Kdim = N = 256
    x, _, _ = O.bitlinear_case(M, Kdim, N, seed=3)
    g = torch.Generator().manual_seed(11)
    ws = [torch.randn(N, Kdim, generator=g) * 0.02 for _ in range(3)]
    nws = [1.0 + 0.1 * torch.randn(Kdim, generator=g) for _ in range(3)]
    pw = K.stack_packed([K.pack_weight(dev(w)) for w in ws])
    qs = [K.act_quant(dev(x), dev(nw), 1e-6) for nw in nws]
    q = torch.cat([t[0] for t in qs]); dq = torch.cat([t[1] for t in qs]); rs = torch.cat([t[2] for t in qs])
    from matmulfreellm_b200 import _lib
    outs = {kernel: K.bitlinear(q, dq, rs, pw, torch.float32, kernel=kernel) for kernel in (K.KERNEL_AUTO, K.KERNEL_GEMV, K.KERNEL_MMA)}
    with _lib.experiments_library():
        outs[K.KERNEL_STREAM] = K.bitlinear(q, dq, rs, pw, torch.float32, kernel=K.KERNEL_STREAM)
    for kernel, out in outs.items():
        for gi in range(3):
            codes, mean = O.ternary_codes(ws[gi])
            ref = O.bitlinear_int(x, nws[gi], codes, mean, 1e-6)[0]
            assert torch.equal(out[:, gi * N:(gi + 1) * N].cpu(), ref), (kernel, gi)


def test_bitlinear_matches_reference_output(K, golden):
    """Against BitLinear.forward of the reference (fp32): agreement to fp32 accuracy."""
    q = golden["quant_cases"]
    for idx, (M, Kd, N, seed) in enumerate(q["cases"]):
        x, nw = torch.from_numpy(q[f"c{idx}_x"]), torch.from_numpy(q[f"c{idx}_nw"])
        _, w, _ = O.bitlinear_case(int(M), int(Kd), int(N), seed=int(seed), dtype=torch.float32)
        pw = K.pack_weight(dev(w))
        qq, dq, rs = K.act_quant(dev(x), dev(nw), 1e-8)
        out = K.bitlinear(qq, dq, rs, pw, torch.float32).cpu().numpy()
        ref = q[f"c{idx}_y"]
        d = np.abs(out - ref)
        # a code flipped at a tie moves one row by <= dq*mean|w| ~ 1e-3 of the output scale
        assert np.quantile(d, 0.5) <= 2e-6 * np.abs(ref).max() and d.max() <= 5e-3 * np.abs(ref).max()


def test_bitlinear_persistent_kernel(K):
    """The persistent large-M tensor-core kernel, forced on (knob 7 = 1: shape chosen by the library; 11..22: each
    compiled shape — 256-token tile with one accumulator, 192-token tile with two accumulators, the same with the
    TMA-store epilogue, separate rings, two issuing threads, the shallow activation ring, the two shapes run by pairs
    of CTAs, and those with the fragment / stmatrix / TMA-store epilogue and with rings eight deep) for problems with a ragged last token tile, a ragged last weight tile and a trailing 64-wide K stage:
    bit-exact accumulators and outputs in all three dtypes against the CUDA-core kernel; the paired shapes refuse a
    projection that is not an even number of whole weight tiles; then a grouped (3 x norm weight) call."""
    from matmulfreellm_b200 import _lib
    with _lib.experiments_library() as lib:      # the build that exports the configuration overrides
        for (M, Kd, N) in [(300, 704, 384), (700, 2048, 512), (1024, 2560, 200), (129, 256, 128), (520, 4096, 256), (900, 704, 768)]:
            x, w, _ = O.bitlinear_case(M, Kd, N, seed=M)
            pw = K.pack_weight(dev(w))
            q, dq, rs = K.act_quant(dev(x), None, 1e-6)
            lib.mmf_tuning(7, 2)
            ref, acc_ref = K.bitlinear(q, dq, rs, pw, torch.float32, kernel=K.KERNEL_GEMV, return_acc=True)
            pairable = N % 256 == 0
            for knob in (1, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22):
                lib.mmf_tuning(7, knob)
                if knob >= 18 and not pairable:
                    with pytest.raises(_lib.MMFreeError) as e:
                        K.bitlinear(q, dq, rs, pw, torch.float32, kernel=K.KERNEL_MMA)
                    assert e.value.code == -2
                    continue
                out, acc = K.bitlinear(q, dq, rs, pw, torch.float32, kernel=K.KERNEL_MMA, return_acc=True)
                K.check_status()
                assert torch.equal(acc, acc_ref) and torch.equal(out, ref), (M, Kd, N, knob)
                for dt in (torch.bfloat16, torch.float16):
                    assert torch.equal(K.bitlinear(q, dq, rs, pw, dt, kernel=K.KERNEL_MMA), ref.to(dt)), (M, Kd, N, knob, dt)
                    got, acc2 = K.bitlinear(q, dq, rs, pw, dt, kernel=K.KERNEL_MMA, return_acc=True)
                    assert torch.equal(got, ref.to(dt)) and torch.equal(acc2, acc_ref), (M, Kd, N, knob, dt)
        M, Kdim, N = 260, 256, 256
        x, _, _ = O.bitlinear_case(M, Kdim, N, seed=3)
        g = torch.Generator().manual_seed(11)
        ws = [torch.randn(N, Kdim, generator=g) * 0.02 for _ in range(3)]
        nws = [1.0 + 0.1 * torch.randn(Kdim, generator=g) for _ in range(3)]
        pw = K.stack_packed([K.pack_weight(dev(w)) for w in ws])
        qs = [K.act_quant(dev(x), dev(nw), 1e-6) for nw in nws]
        q = torch.cat([t[0] for t in qs]); dq = torch.cat([t[1] for t in qs]); rs = torch.cat([t[2] for t in qs])
        for knob in (11, 12, 13, 18, 19, 20, 21, 22):
            lib.mmf_tuning(7, knob)
            for dt in (torch.float32, torch.bfloat16):
                out = K.bitlinear(q, dq, rs, pw, dt, kernel=K.KERNEL_MMA)
                K.check_status()
                for gi in range(3):
                    codes, mean = O.ternary_codes(ws[gi])
                    ref = O.bitlinear_int(x, nws[gi], codes, mean, 1e-6)[0]
                    assert torch.equal(out[:, gi * N:(gi + 1) * N].cpu(), ref.to(dt)), (knob, dt, gi)


def test_bitlinear_large_m_properties(K):
    """4096 token rows (a prompt-sized call): rows are independent, so a slice of a 4096-row call equals the same rows run alone,
    and the first rows match the oracle."""
    M, Kdim, N = 4096, 2048, 2048
    x, w, _ = O.bitlinear_case(M, Kdim, N, seed=9)
    pw = K.pack_weight(dev(w))
    q, dq, rs = K.act_quant(dev(x), None, 1e-6)
    out, acc = K.bitlinear(q, dq, rs, pw, torch.float32, return_acc=True)
    sl = slice(1000, 1016)
    out_s, acc_s = K.bitlinear(q[sl].contiguous(), dq[sl].contiguous(), rs[sl].contiguous(), pw, torch.float32,
                               return_acc=True)
    assert torch.equal(out[sl], out_s) and torch.equal(acc[sl], acc_s)
    codes, mean = O.ternary_codes(w)
    ref, acc_ref, _, _ = O.bitlinear_int(x[:32], None, codes, mean, 1e-6)
    assert np.array_equal(acc[:32].cpu().numpy(), acc_ref) and torch.equal(out[:32].cpu(), ref)
    # column checksum: sum over rows of acc equals (sum of codes rows) . weights, computed in int64
    colsum = q.long().sum(0).cpu().numpy()
    assert np.array_equal(acc.long().sum(0).cpu().numpy(), codes.astype(np.int64) @ colsum)


# ----------------------------------------------------------------------------------------------------------
# HGRN recurrence
# ----------------------------------------------------------------------------------------------------------
def _hgrn_check(K, x, g, h0, log, rtol_o, rtol_h):
    o_ref, ht_ref = (O.chunk_hgrn_ref if log else O.naive_recurrent_hgrn)(x, g, h0, True)
    o, ht = K.hgrn_scan(dev(x), dev(g), None if h0 is None else dev(h0), True, gate_is_log=log,
                        state_dtype=torch.float32)
    so = o_ref.float().abs().max().item()
    assert (o.cpu().float() - o_ref.float()).abs().max().item() <= rtol_o * so
    assert (ht.cpu() - ht_ref).abs().max().item() <= rtol_h * ht_ref.abs().max().item()


def test_hgrn_matches_reference_fixture(K, golden):
    h = golden["hgrn_cases"]
    x, g, h0 = (torch.from_numpy(h[k]) for k in ("x", "g", "h0"))
    o, ht = K.hgrn_scan(dev(x), dev(g), dev(h0), True, gate_is_log=False, state_dtype=torch.float32)
    assert np.abs(o.cpu().numpy() - h["o"]).max() <= 1e-5 and np.abs(ht.cpu().numpy() - h["ht"]).max() <= 1e-5
    o, none = K.hgrn_scan(dev(x), dev(g), None, False, gate_is_log=False)
    assert none is None and np.abs(o.cpu().numpy() - h["o_nostate"]).max() <= 1e-5
    ob, htb = K.hgrn_scan(dev(x).bfloat16(), dev(g).bfloat16(), dev(h0), True, gate_is_log=False,
                          state_dtype=torch.float32)
    # bf16 outputs: one rounding of an fp32 state that matches to 1e-5 -> at most one bf16 ulp (2^-8 relative)
    assert np.abs(ob.float().cpu().numpy() - h["o_bf16"]).max() <= 2 ** -7 * np.abs(h["o_bf16"]).max()
    assert np.abs(htb.cpu().numpy() - h["ht_bf16"]).max() <= 1e-4 * np.abs(h["ht_bf16"]).max()


@pytest.mark.parametrize("B,T,D", [(2, 1, 64), (3, 37, 72), (2, 300, 256), (1, 2048, 128), (8, 512, 2048)])
@pytest.mark.parametrize("log", [False, True])
def test_hgrn_scan_vs_oracle(K, B, T, D, log):
    """fp32 state: rel 1e-4; bf16 outputs: rel 1e-2 (tolerances of the hot-path specification).  (1,2048,128)
    takes the time-chunked two-pass path."""
    x, g_log = O.hgrn_case(B, T, D, seed=B + T, dtype=torch.bfloat16)
    g = g_log if log else torch.exp(g_log)
    h0 = torch.randn(B, 1, D, generator=torch.Generator().manual_seed(1))
    _hgrn_check(K, x, g, h0, log, 1e-2, 1e-4)
    _hgrn_check(K, x.float(), g, None, log, 1e-4, 1e-4)


def test_hgrn_full_size_against_torch_loop(K):
    """B=8, D=2048, T=2048 (the size of the recurrence benchmark) against a plain fp32 PyTorch loop on the same device
    (the CPU oracle checks the same size in tests/test_gpu_full_size.py)."""
    x, g_log = O.hgrn_case(8, 2048, 2048, seed=0, dtype=torch.bfloat16)
    xd, gd = dev(x).squeeze(1), dev(g_log).squeeze(1)
    o, ht = K.hgrn_scan(xd, gd, None, True, gate_is_log=True, state_dtype=torch.float32)
    h = torch.zeros(8, 2048, device="cuda")
    f = torch.exp(gd)
    worst = 0.0
    for t in range(2048):
        h = f[:, t] * h + xd[:, t].float()
        if t % 256 == 255 or t == 2047:
            worst = max(worst, (o[:, t].float() - h).abs().max().item() / h.abs().max().item())
    assert worst <= 1e-2
    assert (ht - h).abs().max().item() <= 1e-4 * h.abs().max().item()
    # decode-shaped call: B=256, T=1, state updated in place
    st = torch.randn(256, 2048, device="cuda")
    x1 = torch.randn(256, 1, 2048, device="cuda").bfloat16()
    g1 = torch.rand(256, 1, 2048, device="cuda")
    want = g1[:, 0] * st + x1[:, 0].float()
    o1, st2 = K.hgrn_scan(x1, g1, st, True, gate_is_log=False, state_dtype=torch.float32, final_state_out=st)
    assert st2.data_ptr() == st.data_ptr()
    assert (st - want).abs().max().item() <= 1e-5 and (o1[:, 0].float() - want).abs().max().item() <= 2e-2


# ----------------------------------------------------------------------------------------------------------
# norms, activations, helpers
# ----------------------------------------------------------------------------------------------------------
def test_norms_match_reference_fixture(K, golden):
    n = golden["norm_cases"]
    x, w, res, og = (dev(torch.from_numpy(n[k])) for k in ("x", "w", "res", "o"))
    assert np.abs(K.rmsnorm(x, w, 1e-6).cpu().numpy() - n["y"]).max() <= 2e-6
    y2, r2 = K.rmsnorm(x, w, 1e-6, residual=res, prenorm=True)
    assert np.abs(y2.cpu().numpy() - n["y_res"]).max() <= 2e-6 and np.array_equal(r2.cpu().numpy(), n["res_out"])
    assert np.abs(K.rmsnorm_swishgate(x, og, w, 1e-6).cpu().numpy() - n["gate"]).max() <= 5e-6
    assert np.abs(K.swiglu(x, og).cpu().numpy() - n["swiglu"]).max() <= 5e-6


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("D", [256, 2048, 100])
def test_rowwise_ops_vs_oracle(K, dtype, D):
    g = torch.Generator().manual_seed(D)
    M = 9
    x = (torch.randn(M, D, generator=g) * 2).to(dtype)
    o = torch.randn(M, D, generator=g).to(dtype)
    res = torch.randn(M, D, generator=g).to(dtype)
    w = 1.0 + 0.1 * torch.randn(D, generator=g)
    tol = 1e-5 if dtype == torch.float32 else (2 ** -7 if dtype == torch.bfloat16 else 2 ** -10)

    def close(a, b):
        return (a.float().cpu() - b.float()).abs().max().item() <= tol * max(1.0, b.float().abs().max().item())

    assert close(K.rmsnorm(dev(x), dev(w), 1e-6), O.rms_norm_ref(x, w, eps=1e-6))
    y, r = K.rmsnorm(dev(x), dev(w), 1e-6, residual=dev(res), prenorm=True)
    y_ref, r_ref = O.rms_norm_ref(x, w, residual=res, eps=1e-6, prenorm=True)
    assert close(y, y_ref) and close(r, r_ref)
    y, r = K.rmsnorm(dev(x), dev(w), 1e-6, residual=dev(res).float(), prenorm=True)      # fp32 residual stream
    assert r.dtype == torch.float32 and close(y, y_ref)
    assert close(K.rmsnorm_swishgate(dev(x), dev(o), dev(w), 1e-6), O.swish_gate_norm_ref(x, o, w, 1e-6))
    assert close(K.swiglu(dev(x), dev(o)), O.swiglu_ref(x, o))


def test_swiglu_on_chunk_views(K):
    y = torch.randn(2, 5, 512, generator=torch.Generator().manual_seed(0)).bfloat16()
    gate, up = dev(y).chunk(2, -1)
    ref = O.swiglu_ref(*y.chunk(2, -1))
    assert (K.swiglu(gate, up).cpu().float() - ref.float()).abs().max().item() <= 2 ** -7 * ref.float().abs().max().item()


def test_argmax_and_embedding(K):
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(7, 32000, generator=g)
    logits[3, 100] = logits[3, 20000] = 50.0          # tie -> first index
    for dt in (torch.float32, torch.bfloat16):
        l = logits.to(dt)
        assert torch.equal(K.argmax_rows(dev(l)).cpu(), l.float().argmax(-1))
    assert K.argmax_rows(dev(logits))[3].item() == 100
    table = torch.randn(1000, 256, generator=g).bfloat16()
    ids = torch.randint(0, 1000, (3, 5), generator=g)
    assert torch.equal(K.embedding(dev(table), dev(ids)).cpu(), table[ids])


# ----------------------------------------------------------------------------------------------------------
# fused producers of BitLinear inputs (the kernels between two contractions of a block)
# ----------------------------------------------------------------------------------------------------------
def _codes_close(q, dq, q_ref, dq_ref, exact):
    """exact: bit-identical codes and scales.  Otherwise (a sigmoid / exp sits upstream, whose last-ulp result may
    round an activation to the neighbouring bf16 value): scales agree to 1e-2, codes differ by at most 1 level
    on at most 0.5% of the entries."""
    q, dq = q.cpu().numpy().astype(np.int32), dq.cpu().numpy()
    if exact:
        assert np.array_equal(q, q_ref) and np.array_equal(dq, dq_ref)
    else:
        assert np.allclose(dq, dq_ref, rtol=1e-2)
        d = np.abs(q - q_ref.astype(np.int32))
        assert d.max() <= 1 and (d != 0).mean() <= 5e-3, (d.max(), (d != 0).mean())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_prenorm_quant_bit_exact(K, dtype):
    g = torch.Generator().manual_seed(21)
    M, D = 6, 704
    x = (torch.randn(M, D, generator=g) * 2).to(dtype)
    res = torch.randn(M, D, generator=g).to(dtype)
    nw = 1.0 + 0.1 * torch.randn(D, generator=g)
    bl = [1.0 + 0.1 * torch.randn(D, generator=g) for _ in range(3)]
    # (a) attn_norm -> i/f/g prologues, no residual
    y_ref = O.rms_norm_ref(x, nw, eps=1e-6)
    q, dq, rs, res_out, y = K.prenorm_quant(dev(x), None, dev(nw), 1e-6, [dev(b) for b in bl], 1e-6, False, want_y=True)
    assert res_out is None
    # RMSNorm output: fp64-accumulated statistics on the GPU, fp32 in torch -> allow one rounding step of dtype
    assert (y.cpu().float() - y_ref.float()).abs().max() <= (2 ** -7 if dtype == torch.bfloat16 else 1e-6) * y_ref.float().abs().max()
    for gi in range(3):   # the codes are exact functions of the GPU's own normed row
        q_ref, dq_ref, rs_ref = O.act_codes(y.cpu(), bl[gi], 1e-6)
        assert np.array_equal(q[gi * M:(gi + 1) * M].cpu().numpy(), q_ref)
        assert np.array_equal(dq[gi * M:(gi + 1) * M].cpu().numpy(), dq_ref)
        assert np.array_equal(rs[gi * M:(gi + 1) * M].cpu().numpy(), rs_ref)
    # (b) mlp_norm: fused residual add, statistics on the unrounded sum, residual_out rounded
    y_ref, r_ref = O.rms_norm_ref(x, nw, residual=res, eps=1e-6, prenorm=True)
    q, dq, rs, res_out, y = K.prenorm_quant(dev(x), dev(res), dev(nw), 1e-6, [dev(bl[0])], 1e-6, False,
                                            want_residual_out=True, want_y=True)
    assert torch.equal(res_out.cpu(), r_ref)
    q_ref, dq_ref, _ = O.act_codes(y.cpu(), bl[0], 1e-6)
    assert np.array_equal(q.cpu().numpy(), q_ref) and np.array_equal(dq.cpu().numpy(), dq_ref)
    # (c) next block's attn_norm: the sum is a tensor of its own in the reference -> rounded before the statistics
    h = x + res
    y_ref = O.rms_norm_ref(h, nw, eps=1e-6)
    q, dq, rs, res_out, y = K.prenorm_quant(dev(x), dev(res), dev(nw), 1e-6, [], 1e-6, True, want_residual_out=True,
                                            want_y=True)
    assert q is None and torch.equal(res_out.cpu(), h)
    assert (y.cpu().float() - y_ref.float()).abs().max() <= (2 ** -7 if dtype == torch.bfloat16 else 1e-6) * y_ref.float().abs().max()
    # strided rows (last position of every sequence)
    x3 = dev(x).view(2, 3, D)
    q2, dq2, _, _, _ = K.prenorm_quant(x3[:, -1], None, dev(nw), 1e-6, [dev(bl[0])], 1e-6, False)
    qa, dqa, _, _, _ = K.prenorm_quant(x3[:, -1].contiguous(), None, dev(nw), 1e-6, [dev(bl[0])], 1e-6, False)
    assert torch.equal(q2, qa) and torch.equal(dq2, dqa)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gatenorm_and_swiglu_quant(K, dtype):
    g = torch.Generator().manual_seed(22)
    M, D = 5, 256
    ifg = (torch.randn(M, 3 * D, generator=g)).to(dtype)
    o = torch.randn(M, D, generator=g).to(dtype)
    gw = 1.0 + 0.1 * torch.randn(D, generator=g)
    nw = 1.0 + 0.1 * torch.randn(D, generator=g)
    y_ref = O.swish_gate_norm_ref(ifg[:, 2 * D:], o, gw, 1e-6)
    q_ref, dq_ref, _ = O.act_codes(y_ref, nw, 1e-6)
    q, dq, rs = K.gatenorm_quant(dev(ifg)[:, 2 * D:], dev(o), dev(gw), 1e-6, dev(nw), 1e-6)
    _codes_close(q, dq, q_ref, dq_ref, exact=False)
    assert np.array_equal(rs.cpu().numpy(), q.cpu().numpy().astype(np.int32).sum(-1))
    gu = torch.randn(M, 2 * 704, generator=g).to(dtype)
    nw2 = 1.0 + 0.1 * torch.randn(704, generator=g)
    z_ref = O.swiglu_ref(gu[:, :704], gu[:, 704:])
    q_ref, dq_ref, _ = O.act_codes(z_ref, nw2, 1e-6)
    q, dq, rs = K.swiglu_quant(dev(gu), dev(nw2), 1e-6)
    _codes_close(q, dq, q_ref, dq_ref, exact=False)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 1e-2), (torch.float32, 1e-4)])
@pytest.mark.parametrize("B,T,D", [(3, 1, 256), (2, 70, 128), (2, 200, 64)])
def test_hgrn_gated_with_padding_mask(K, dtype, tol, B, T, D):
    """Left padding: at masked positions the input gate is zeroed (layers/hgrn_bit.py:119-120), fused into the scan."""
    g = torch.Generator().manual_seed(B * 1000 + T)
    ifg = torch.randn(B, T, 3 * D, generator=g).to(dtype)
    h0 = torch.randn(B, D, generator=g)
    mask = torch.ones(B, T, dtype=torch.uint8)
    for b in range(B):
        mask[b, : (b * 37) % max(T // 2, 1) if T > 1 else b % 2] = 0
    f = ifg[..., D:2 * D].sigmoid()
    i = O.swiglu_ref(ifg[..., :D], 1 - f) * mask.unsqueeze(-1).to(dtype)
    o_ref, ht_ref = O.naive_recurrent_hgrn(i.unsqueeze(1), f.unsqueeze(1), h0.unsqueeze(1), True)
    state = dev(h0.clone())
    d_ifg = dev(ifg)
    o = K.hgrn_gated(d_ifg[..., :D], d_ifg[..., D:2 * D], None, state, mask=dev(mask))
    so = o_ref.float().abs().max().item()
    assert (o.cpu().float() - o_ref.squeeze(1).float()).abs().max().item() <= tol * so
    assert (state.cpu() - ht_ref.squeeze(1)).abs().max().item() <= max(tol, 1e-4) * ht_ref.abs().max().item()
    # an all-ones mask changes nothing
    s1, s2 = dev(h0.clone()), dev(h0.clone())
    o1 = K.hgrn_gated(d_ifg[..., :D], d_ifg[..., D:2 * D], None, s1, mask=dev(torch.ones(B, T, dtype=torch.uint8)))
    o2 = K.hgrn_gated(d_ifg[..., :D], d_ifg[..., D:2 * D], None, s2)
    assert torch.equal(o1, o2) and torch.equal(s1, s2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_prenorm_quant_codes_exact_at_scale(K, dtype):
    """6 million codes against the oracle.  A product that is rounded once instead of twice (a multiply merged with the
    add that follows it) changes about one code in 260 000, which the small cases above cannot see."""
    g = torch.Generator().manual_seed(77)
    M, D = 1024, 2048
    x = (torch.randn(M, D, generator=g) * 2).to(dtype)
    nw = 1.0 + 0.1 * torch.randn(D, generator=g)
    bl = [1.0 + 0.1 * torch.randn(D, generator=g) for _ in range(3)]
    q, dq, rs, _, y = K.prenorm_quant(dev(x), None, dev(nw), 1e-6, [dev(b) for b in bl], 1e-6, False, want_y=True)
    y = y.cpu()
    for gi in range(3):
        q_ref, dq_ref, rs_ref = O.act_codes(y, bl[gi], 1e-6)
        assert np.array_equal(q[gi * M:(gi + 1) * M].cpu().numpy(), q_ref)
        assert np.array_equal(dq[gi * M:(gi + 1) * M].cpu().numpy(), dq_ref)
        assert np.array_equal(rs[gi * M:(gi + 1) * M].cpu().numpy(), rs_ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("D", [704, 2048, 2560, 5632, 6912])
def test_fused_row_kernels_many_rows(K, dtype, D):
    """With more rows than resident CTAs the fused row kernels run their second build: CTAs loop over rows and fetch
    the next row into shared memory while they work.  Rows are independent, so a 1500-row call must reproduce, bit for
    bit, the same rows run in 250-row calls, which take the one-CTA-per-row build that the cases above check against
    the oracle."""
    g = torch.Generator().manual_seed(D)
    M = 1500
    x = dev((torch.randn(M, D, generator=g) * 2).to(dtype))
    res = dev(torch.randn(M, D, generator=g).to(dtype))
    nw = dev(1.0 + 0.1 * torch.randn(D, generator=g))
    bl = [dev(1.0 + 0.1 * torch.randn(D, generator=g)) for _ in range(3)]
    parts = [slice(i, i + 250) for i in range(0, M, 250)]

    def check(fn, n_groups):
        big = fn(slice(0, M))
        small = [fn(sl) for sl in parts]
        for k, t in enumerate(big):
            if t is None:
                continue
            if n_groups > 1 and t.shape[0] == n_groups * M:       # group-major codes / scales
                t = t.view(n_groups, M, *t.shape[1:])
                ref = torch.cat([sm[k].view(n_groups, -1, *t.shape[2:]) for sm in small], dim=1)
            else:
                ref = torch.cat([sm[k] for sm in small], dim=0)
            assert torch.equal(t, ref), (k, D, dtype)

    check(lambda sl: K.prenorm_quant(x[sl], res[sl], nw, 1e-6, bl, 1e-6, False, want_residual_out=True, want_y=True), 3)
    check(lambda sl: K.prenorm_quant(x[sl], None, nw, 1e-6, [bl[0]], 1e-6, True), 1)
    check(lambda sl: K.gatenorm_quant(x[sl], res[sl], nw, 1e-6, bl[1], 1e-6), 1)
    gu = dev(torch.randn(M, 2 * D, generator=g).to(dtype))
    check(lambda sl: K.swiglu_quant(gu[sl], bl[2], 1e-6), 1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("D", [512, 704, 2048, 2560])
def test_fused_row_kernels_four_rows_per_cta(K, dtype, D):
    """From 3072 rows on, rows of at most 2048 values are worked on four at a time per CTA (64 threads and up to 32 values
    per thread each), rows of at most 4096 values two at a time.  A 4099-row call (ragged against the four row slots) must reproduce, bit for bit, the same rows run in
    250-row calls (one CTA per row, checked against the oracle above); the codes of the three-projection call are also
    compared with the oracle directly."""
    g = torch.Generator().manual_seed(D + 1)
    M = 4099
    x = dev((torch.randn(M, D, generator=g) * 2).to(dtype))
    res = dev(torch.randn(M, D, generator=g).to(dtype))
    nw = dev(1.0 + 0.1 * torch.randn(D, generator=g))
    bl = [dev(1.0 + 0.1 * torch.randn(D, generator=g)) for _ in range(3)]
    parts = [slice(i, min(M, i + 250)) for i in range(0, M, 250)]

    def check(fn, n_groups):
        big = fn(slice(0, M))
        small = [fn(sl) for sl in parts]
        for k, t in enumerate(big):
            if t is None:
                continue
            if n_groups > 1 and t.shape[0] == n_groups * M:       # group-major codes / scales
                t = t.view(n_groups, M, *t.shape[1:])
                ref = torch.cat([sm[k].view(n_groups, -1, *t.shape[2:]) for sm in small], dim=1)
            else:
                ref = torch.cat([sm[k] for sm in small], dim=0)
            assert torch.equal(t, ref), (k, D, dtype)
        return big

    q, dq, rs, _, y = check(lambda sl: K.prenorm_quant(x[sl], res[sl], nw, 1e-6, bl, 1e-6, False, want_residual_out=True, want_y=True), 3)
    for gi in range(3):
        q_ref, dq_ref, rs_ref = O.act_codes(y.cpu(), bl[gi].cpu(), 1e-6)
        assert np.array_equal(q[gi * M:(gi + 1) * M].cpu().numpy(), q_ref)
        assert np.array_equal(dq[gi * M:(gi + 1) * M].cpu().numpy(), dq_ref)
        assert np.array_equal(rs[gi * M:(gi + 1) * M].cpu().numpy(), rs_ref)
    check(lambda sl: K.prenorm_quant(x[sl], None, nw, 1e-6, [bl[0]], 1e-6, True), 1)
    check(lambda sl: K.prenorm_quant(x[sl], res[sl], nw, 1e-6, [], 1e-6, True, want_residual_out=True, want_y=True), 0)
    check(lambda sl: K.gatenorm_quant(x[sl], res[sl], nw, 1e-6, bl[1], 1e-6), 1)
    gu = dev(torch.randn(M, 2 * D, generator=g).to(dtype))
    check(lambda sl: K.swiglu_quant(gu[sl], bl[2], 1e-6), 1)
    K.check_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("D", [5632, 6912])
def test_swiglu_quant_two_rows_per_cta(K, dtype, D):
    """Rows of the MLP width on a prompt: two rows per CTA, 128 threads and up to 56 values per thread each; a 3100-row
    call equals the same rows run in 250-row calls bit for bit, and the first rows match the oracle's codes."""
    g = torch.Generator().manual_seed(D)
    M = 3100
    gu = dev(torch.randn(M, 2 * D, generator=g).to(dtype))
    nw = dev(1.0 + 0.1 * torch.randn(D, generator=g))
    q, dq, rs = K.swiglu_quant(gu, nw, 1e-6)
    for i in range(0, M, 250):
        qs, dqs, rss = K.swiglu_quant(gu[i:i + 250], nw, 1e-6)
        assert torch.equal(q[i:i + 250], qs) and torch.equal(dq[i:i + 250], dqs) and torch.equal(rs[i:i + 250], rss), i
    z_ref = O.swiglu_ref(gu[:64, :D].cpu(), gu[:64, D:].cpu())
    q_ref, dq_ref, _ = O.act_codes(z_ref, nw.cpu(), 1e-6)
    _codes_close(q[:64], dq[:64], q_ref, dq_ref, exact=False)
    K.check_status()


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 1e-2), (torch.float32, 1e-4)])
@pytest.mark.parametrize("B,T,D", [(3, 1, 256), (2, 70, 128), (1, 1024, 64)])
def test_hgrn_gated_vs_oracle(K, dtype, tol, B, T, D):
    """The attention layer's gate glue + recurrence (layers/hgrn_bit.py:113-125) in one kernel, state in place."""
    g = torch.Generator().manual_seed(B * 100 + T)
    ifg = torch.randn(B, T, 3 * D, generator=g).to(dtype)
    lb = (torch.rand(D, generator=g) * 0.5).to(dtype)
    h0 = torch.randn(B, D, generator=g)
    for bound in (lb, None):
        f = ifg[..., D:2 * D].sigmoid()
        if bound is not None:
            f = bound + (1 - bound) * f
        i = O.swiglu_ref(ifg[..., :D], 1 - f)
        o_ref, ht_ref = O.naive_recurrent_hgrn(i.unsqueeze(1), f.unsqueeze(1), h0.unsqueeze(1), True)
        state = dev(h0.clone())
        d_ifg = dev(ifg)
        o = K.hgrn_gated(d_ifg[..., :D], d_ifg[..., D:2 * D], None if bound is None else dev(bound), state)
        so = o_ref.float().abs().max().item()
        assert (o.cpu().float() - o_ref.squeeze(1).float()).abs().max().item() <= tol * so
        assert (state.cpu() - ht_ref.squeeze(1)).abs().max().item() <= max(tol, 1e-4) * ht_ref.abs().max().item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,D", [(1, 256), (5, 2048), (3, 2560)])
def test_decode_mix_equals_scan_plus_gatenorm(K, dtype, M, D):
    """The one-kernel decode step is the T = 1 case of hgrn_gated followed by gatenorm_quant: identical codes and
    identical state."""
    g = torch.Generator().manual_seed(M + D)
    ifg = dev(torch.randn(M, 3 * D, generator=g).to(dtype))
    lb = dev((torch.rand(D, generator=g) * 0.5).to(dtype))
    h0 = dev(torch.randn(M, D, generator=g))
    gw = dev(1.0 + 0.1 * torch.randn(D, generator=g))
    nw = dev(1.0 + 0.1 * torch.randn(D, generator=g))
    for bound in (lb, None):
        s1, s2 = h0.clone(), h0.clone()
        v = ifg.view(M, 1, 3 * D)
        o = K.hgrn_gated(v[..., :D], v[..., D:2 * D], bound, s1)
        q1, dq1, rs1 = K.gatenorm_quant(ifg[:, 2 * D:], o.view(M, D), gw, 1e-6, nw, 1e-6)
        q2, dq2, rs2 = K.decode_mix(ifg, bound, s2, gw, 1e-6, nw, 1e-6)
        assert torch.equal(s1, s2) and torch.equal(q1, q2) and torch.equal(dq1, dq2) and torch.equal(rs1, rs2)


def test_bitlinear_mma_configurations_agree(K):
    """Every configuration the tensor-core kernel can be tuned into (K split over clusters of 2/4/8, the deep ring,
    128- or 256-token tiles, two weight tiles per CTA) gives the same int32 accumulators as the CUDA-core kernel."""
    from matmulfreellm_b200 import _lib
    with _lib.experiments_library() as lib:      # the build that exports the configuration overrides
        for (M, Kd, N) in [(32, 2048, 2048), (40, 704, 384), (300, 2048, 512), (9, 2048, 200), (70, 2048, 256), (128, 5632, 128)]:
            x, w, _ = O.bitlinear_case(M, Kd, N, seed=M)
            pw = K.pack_weight(dev(w))
            q, dq, rs = K.act_quant(dev(x), None, 1e-6)
            ref, acc_ref = K.bitlinear(q, dq, rs, pw, torch.float32, kernel=K.KERNEL_GEMV, return_acc=True)
            # knob 10 = split-K partial sums by st.async + the owner's mbarrier (1 = on, 2 = off), tried with every K split
            for knob, values in ((0, (1, 2, 4, 8)), (2, (1,)), (1, (128, 256)), (3, (2,)), (10, (2, 4, 8, 0))):
                for v in values:
                    if knob == 10:
                        lib.mmf_tuning(10, 1)
                        lib.mmf_tuning(0, v)
                    else:
                        lib.mmf_tuning(knob, v)
                    if knob == 3:
                        lib.mmf_tuning(1, 128)
                    try:
                        out, acc = K.bitlinear(q, dq, rs, pw, torch.float32, kernel=K.KERNEL_MMA, return_acc=True)
                    except _lib.MMFreeError as e:      # a forced combination that does not exist for this shape
                        assert e.code == -2
                        continue
                    finally:
                        for kk in range(11):
                            lib.mmf_tuning(kk, 0)
                    K.check_status()
                    assert torch.equal(acc, acc_ref) and torch.equal(out, ref), (M, Kd, N, knob, v)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("temperature,top_p", [(1.0, 1.0), (0.6, 0.4), (2.0, 0.9), (1.0, 0.0)])
def test_sample_top_p_vs_oracle(K, dtype, temperature, top_p):
    """Temperature + nucleus sampling with supplied uniform numbers equals the oracle's inverse-CDF draw on every row
    whose draw is not within 2e-6 (of the total mass) of a CDF step — there the last bits of the exponentials decide."""
    g = torch.Generator().manual_seed(int(temperature * 10 + top_p * 100))
    M, V = 48, 32000
    logits = (torch.randn(M, V, generator=g) * 3).to(dtype)
    logits[0, 5:9] = logits[0].max() + 1          # a tie among the most probable tokens
    u = torch.rand(M, generator=g)
    u[1] = 0.0
    ref, margin = O.sample_top_p_ref(logits.float().numpy(), temperature, top_p, u.numpy())
    got = K.sample_top_p(dev(logits), temperature, top_p, dev(u)).cpu().numpy()
    safe = margin > 2e-6
    assert safe.mean() > 0.5 and np.array_equal(got[safe], ref[safe])
    if top_p == 0.0:                              # degenerates to arg-max (one of the tied maxima, chosen by u)
        lf = logits.float()
        assert torch.equal(lf[torch.arange(M), torch.from_numpy(got)], lf.max(-1).values)
    # same inputs, same tokens
    again = K.sample_top_p(dev(logits), temperature, top_p, dev(u)).cpu().numpy()
    assert np.array_equal(got, again)


@pytest.mark.parametrize("gate_is_log", [True, False])
def test_time_sliced_scan_stitches_to_whole_scan(K, gate_is_log):
    """The exchange of the sequence-sharded scan, with the ranks emulated one after the other on one GPU: every
    slice is reduced to (decay, final state), the pairs are folded, slices after the first are run again from their
    incoming state.  Outputs and the final state must equal the scan over the whole sequence (fp32 state 1e-4)."""
    from matmulfreellm_b200.seq_sharding import fold_carries, slice_decay
    g = torch.Generator().manual_seed(31)
    B, T, D = 2, 3000, 128
    x = dev(torch.randn(B, T, D, generator=g).to(torch.bfloat16))
    gl = torch.nn.functional.logsigmoid(torch.randn(B, T, D, generator=g) + 2.0)
    gate = dev(gl if gate_is_log else gl.exp())
    h0 = dev(torch.randn(B, D, generator=g))
    o_ref, h_ref = K.hgrn_scan(x, gate, h0, True, gate_is_log=gate_is_log, state_dtype=torch.float32)
    cuts = [(0, 1000), (1000, 1001), (1001, 2200), (2200, T)]
    first = [K.hgrn_scan(x[:, a:b].contiguous(), gate[:, a:b].contiguous(), h0 if i == 0 else None, True,
                         gate_is_log=gate_is_log, state_dtype=torch.float32) for i, (a, b) in enumerate(cuts)]
    decay = torch.stack([slice_decay(gate[:, a:b], gate_is_log) for a, b in cuts])
    carry, last = fold_carries(decay, torch.stack([f[1] for f in first]))
    outs = [first[0][0]] + [K.hgrn_scan(x[:, a:b].contiguous(), gate[:, a:b].contiguous(), carry[i].contiguous(), True,
                                        gate_is_log=gate_is_log, state_dtype=torch.float32)[0]
                            for i, (a, b) in enumerate(cuts) if i > 0]
    o = torch.cat(outs, dim=1)
    assert (o.float() - o_ref.float()).abs().max().item() <= 1e-2 * o_ref.float().abs().max().item()
    assert (last - h_ref).abs().max().item() <= 1e-4 * h_ref.abs().max().item()
