"""Pin the CPU oracle against fixtures produced by running the reference itself
(tests/golden/make_golden.py).  No GPU needed."""
import numpy as np
import pytest
import torch

from oracle import mmfree_oracle as O


def t(a):
    return torch.from_numpy(np.asarray(a))


def test_fixture_inputs_regenerate(golden):
    """The seeded latent weights the fixtures were made from come out of the generator unchanged."""
    q = golden["quant_cases"]
    for idx, (M, K, N, seed) in enumerate(q["cases"]):
        x, w, _ = O.bitlinear_case(int(M), int(K), int(N), seed=int(seed), dtype=torch.float32)
        assert np.array_equal(x.numpy(), q[f"c{idx}_x"])
        assert w.double().sum().item() == q[f"c{idx}_w_sum"]
        assert w.double().abs().sum().item() == q[f"c{idx}_w_abs_sum"]


def test_float_restatements_match_reference(golden):
    q = golden["quant_cases"]
    for idx, (M, K, N, seed) in enumerate(q["cases"]):
        x = t(q[f"c{idx}_x"])
        _, w, _ = O.bitlinear_case(int(M), int(K), int(N), seed=int(seed), dtype=torch.float32)
        nw = t(q[f"c{idx}_nw"])
        xn = O.rms_norm_ref(x, nw, eps=1e-8)
        assert torch.equal(xn, t(q[f"c{idx}_xn"]))
        assert torch.equal(O.activation_quant(xn), t(q[f"c{idx}_actq"]))
        wq_ref = t(q[f"c{idx}_wq_sign"]).float() * t(q[f"c{idx}_wq_mag"])
        assert torch.equal(O.weight_quant(w), wq_ref)
        assert torch.equal(O.bitlinear_ref(x, nw, w, eps=1e-8), t(q[f"c{idx}_y"]))


def test_integer_restatement_matches_reference(golden):
    """Ternary codes equal sign(weight_quant(w)); activation codes equal activation_quant*scale except where
    the reference's pre-rounding value sits within 1e-3 of a tie (its row sum is accumulated in fp32, the
    oracle's in fp64); the dequantised product matches the reference output to fp32 accuracy."""
    q = golden["quant_cases"]
    for idx, (M, K, N, seed) in enumerate(q["cases"]):
        x = t(q[f"c{idx}_x"])
        _, w, _ = O.bitlinear_case(int(M), int(K), int(N), seed=int(seed), dtype=torch.float32)
        nw = t(q[f"c{idx}_nw"])
        codes, mean = O.ternary_codes(w)
        assert np.array_equal(codes, q[f"c{idx}_wq_sign"])
        assert abs(float(mean) - float(q[f"c{idx}_wq_mag"])) <= 1.2e-7 * float(mean)

        qx, dq, rowsum = O.act_codes(x, nw, eps=1e-8)
        xn = q[f"c{idx}_xn"]
        s = np.float32(127.0) / np.maximum(np.abs(xn).max(-1, keepdims=True), np.float32(1e-5))
        ref_codes = np.rint(q[f"c{idx}_actq"] * s)
        pre = xn * s
        diff = qx != ref_codes
        near_tie = np.abs(np.abs(pre - np.floor(pre)) - 0.5) < 1e-3
        assert np.all(~diff | near_tie), "activation codes differ away from rounding ties"
        assert diff.sum() <= 2
        assert np.array_equal(rowsum, qx.astype(np.int64).sum(-1))

        out, acc, _, _ = O.bitlinear_int(x, nw, codes, mean, eps=1e-8)
        ref = q[f"c{idx}_y"]
        assert np.abs(out.numpy() - ref).max() <= 2e-6 * np.abs(ref).max()
        assert np.abs(acc).max() < 2 ** 24


def test_pack_layout_roundtrip():
    rng = np.random.default_rng(0)
    codes = rng.integers(-1, 2, size=(200, 192)).astype(np.int8)     # N not a multiple of 128
    words = O.pack_ternary(codes)
    assert words.size == 2 * 3 * 128 * 4
    KC = 3
    for (n, k) in [(0, 0), (5, 17), (127, 191), (128, 64), (199, 100)]:
        tile, r, c, qd, j = n // 128, n % 128, k // 64, (k % 64) // 16, k % 16
        word = int(words[((tile * KC + c) * 128 + r) * 4 + qd])
        f = j // 4 + 4 * (j % 4)
        assert ((word >> (2 * f)) & 3) - 1 == codes[n, k]
    # padding rows hold code 0 (field value 1)
    assert words[((1 * KC + 0) * 128 + 100) * 4] == 0x55555555


def test_hgrn_and_norms_match_reference(golden):
    h = golden["hgrn_cases"]
    o, ht = O.naive_recurrent_hgrn(t(h["x"]), t(h["g"]), t(h["h0"]), True)
    assert torch.equal(o, t(h["o"])) and torch.equal(ht, t(h["ht"]))
    o0, none = O.naive_recurrent_hgrn(t(h["x"]), t(h["g"]), None, False)
    assert none is None and torch.equal(o0, t(h["o_nostate"]))
    ob, htb = O.naive_recurrent_hgrn(t(h["x"]).bfloat16(), t(h["g"]).bfloat16(), t(h["h0"]), True)
    assert torch.equal(ob.float(), t(h["o_bf16"])) and torch.equal(htb, t(h["ht_bf16"]))
    # chunk_hgrn's log-gate convention is the same recurrence
    oc, _ = O.chunk_hgrn_ref(t(h["x"]), torch.log(t(h["g"])), t(h["h0"]), True)
    assert torch.allclose(oc, t(h["o"]), rtol=1e-5, atol=1e-6)

    n = golden["norm_cases"]
    x, w, res, og = t(n["x"]), t(n["w"]), t(n["res"]), t(n["o"])
    assert torch.equal(O.rms_norm_ref(x, w, eps=1e-6), t(n["y"]))
    y2, r2 = O.rms_norm_ref(x, w, residual=res, eps=1e-6, prenorm=True)
    assert torch.equal(y2, t(n["y_res"])) and torch.equal(r2, t(n["res_out"]))
    assert torch.allclose(O.swish_gate_norm_ref(x, og, w, eps=1e-6), t(n["gate"]), rtol=1e-6, atol=1e-7)
    assert torch.allclose(O.swiglu_ref(x, og), t(n["swiglu"]), rtol=1e-6, atol=1e-7)


def _tiny(golden, linear):
    g = golden["tiny_model"]
    cfg = O.OracleConfig(vocab_size=32000, hidden_size=256, num_hidden_layers=2, intermediate_size=704)
    sd = O.random_weights(cfg, seed=0)
    sd["model.lower_bounds"] = t(g["lower_bounds"])
    return g, cfg, sd, O.OracleHGRNBit(cfg, sd, dtype=torch.float32, linear=linear, bitlinear_eps=1e-8)


def _close_up_to_code_flips(got, ref, typical, worst):
    """Quantisation is discontinuous: an fp32-ulp difference upstream flips an occasional int8 code and
    moves that token's outputs by ~dq*mean|w|.  So: almost every element agrees to `typical`, and none is
    further off than `worst` (both relative to max|ref|)."""
    scale = np.abs(ref).max()
    d = np.abs(got - ref)
    assert np.quantile(d, 0.5) <= typical * scale, np.quantile(d, 0.5) / scale
    assert d.max() <= worst * scale, d.max() / scale


def test_tiny_model_float_path_matches_reference(golden):
    g, cfg, sd, model = _tiny(golden, "float")
    assert sorted(sd.keys()) == list(g["state_dict_keys"])
    ids = t(g["ids"])
    logits, states = model.forward(ids)
    _close_up_to_code_flips(logits[:, g["logits_pos"]].numpy(), g["logits_at"], 1e-6, 2e-3)
    assert (logits.argmax(-1).numpy() == g["argmax"]).mean() >= 0.99
    assert np.abs(logits.double().sum(-1).numpy() - g["logits_sum"]).max() <= 1e-3 * g["logits_abs_sum"].max()
    for i, s in enumerate(states):
        _close_up_to_code_flips(s.numpy(), g["states"][i], 1e-6, 2e-3)


def test_tiny_model_integer_path_matches_reference(golden):
    g, cfg, sd, model = _tiny(golden, "int")
    ids = t(g["ids"])
    logits, states = model.forward(ids)
    _close_up_to_code_flips(logits[:, g["logits_pos"]].numpy(), g["logits_at"], 2e-5, 5e-2)
    for i, s in enumerate(states):
        _close_up_to_code_flips(s.numpy(), g["states"][i], 2e-5, 5e-2)
    assert (logits.argmax(-1).numpy() == g["argmax"]).mean() >= 0.95   # near-flat logits of a random-init model
    toks, margins = model.greedy(ids, 16)
    same = toks.numpy() == g["greedy_tokens"]
    # a sequence may only leave the reference's greedy path at a step whose top-2 margin is within the
    # code-flip noise (5e-3 of the logit scale ~1)
    for b in range(same.shape[0]):
        if not same[b].all():
            first = int(np.argmin(same[b]))
            assert g["greedy_margins"][b, first] < 5e-3, (b, first, g["greedy_margins"][b, first])


@pytest.mark.parametrize("temperature,top_p", [(0.6, 0.4), (1.0, 0.9), (2.0, 0.95), (0.7, 1.0)])
def test_nucleus_oracle_matches_transformers_warpers(temperature, top_p):
    """The reference samples through transformers (generate.py:11: do_sample, top_p, temperature).  The oracle's
    tempered-softmax + top-p restatement is pinned here against the library's own TemperatureLogitsWarper and
    TopPLogitsWarper on seeded logits: identical kept sets, renormalised probabilities equal to fp32 accuracy, and
    the inverse-CDF draw over the library's probabilities picks the oracle's token."""
    from transformers.generation.logits_process import TemperatureLogitsWarper, TopPLogitsWarper
    g = torch.Generator().manual_seed(int(temperature * 100 + top_p * 1000))
    M, V = 24, 32000
    logits = torch.randn(M, V, generator=g) * 3
    u = torch.rand(M, generator=g).numpy()
    scores = TemperatureLogitsWarper(temperature)(None, logits.clone())
    if top_p < 1.0:
        scores = TopPLogitsWarper(top_p)(None, scores)
    kept_hf = torch.isfinite(scores).numpy()
    probs_hf = torch.softmax(scores.double(), -1).numpy()
    kept, w, margin = O.nucleus_ref(logits.numpy(), temperature, top_p)
    tok, draw_margin = O.sample_top_p_ref(logits.numpy(), temperature, top_p, u)
    n_same = 0
    for m in range(M):
        # the library takes its cumulative sum in fp32 over up to 32000 terms (error up to ~1e-5 of the mass), so at a
        # flat boundary its kept set may differ from the fp64 one by tokens whose cumulative mass is that close to top_p
        diff = np.nonzero(kept[m] != kept_hf[m])[0]
        if len(diff):
            order = np.argsort(-w[m], kind="stable")
            before = np.concatenate([[0.0], np.cumsum(w[m][order])[:-1]])      # mass of the strictly more probable tokens
            pos = np.empty(V, dtype=np.int64)
            pos[order] = np.arange(V)
            total = w[m].sum()
            assert np.all(np.abs(before[pos[diff]] - top_p * total) <= 2e-5 * total), (m, len(diff))
        # tempered-softmax weights: renormalised over the library's kept set they are the library's probabilities
        p = np.where(kept_hf[m], w[m], 0.0)
        p /= p.sum()
        assert np.allclose(p, probs_hf[m], rtol=2e-5, atol=1e-12), m
        if len(diff) == 0:
            n_same += 1
            if draw_margin[m] > 1e-6:
                c = np.cumsum(probs_hf[m])
                assert int(np.searchsorted(c, u[m] * c[-1], side="right")) == tok[m], m
    assert n_same >= M // 2          # identical kept sets on most rows (all rows at the reference's 0.6 / 0.4 setting)
    if (temperature, top_p) == (0.6, 0.4):
        assert n_same == M
