"""The quantisers in front of the path. CPU: the oracle's restatement of the harness's host rule (tests/gpu/ref_host.cpp:239-258) turns the
`normal` generator's unquantised samples into exactly the generator's bytes. GPU: the device quantisers, through the C ABI, equal that
restatement bit for bit, edge cases included, and their output drives the attention kernels through the usual gate."""
import numpy as np
import pytest


@pytest.mark.parametrize("shape", [(1, 2, 256, 512, 2), (2, 4, 77, 130, 1), (1, 8, 64, 64, 8)], ids=lambda s: "B%dH%dS%dSK%dHK%d" % s)
def test_oracle_quantiser_reproduces_the_generator_bytes(oracle, shape):
    B, H, S, SK, HK = shape
    inp = oracle.generate("normal", B, H, S, SK, HK)
    q, k, v = oracle.generate_raw_normal(B, H, S, SK, HK)
    qb, qs = oracle.quantize_rows(q)          # the generator folds the softmax scale into its Q samples before quantising
    kb, ks = oracle.quantize_rows(k)
    vb, vd = oracle.quantize_tensor(v)
    assert np.array_equal(qb.reshape(inp.q.shape), inp.q) and np.array_equal(qs.ravel(), inp.qs[: qs.size])
    assert np.array_equal(kb.reshape(inp.k.shape), inp.k) and np.array_equal(ks.ravel(), inp.ks[: ks.size])
    assert np.array_equal(vb.reshape(inp.v.shape), inp.v) and vd == np.float32(inp.vdescale)


def test_oracle_quantiser_edge_cases(oracle):
    x = np.zeros((4, 128), np.float32)
    x[1, :32] = 448.0          # amax = 448 = 1.75 * 2^8: scale 2^0, top element exactly representable
    x[1, 32:64] = 449.0        # scale still 2^0: saturates to 448
    x[2, 0] = 2.0 ** -140      # subnormal maximum: scale clamps at E8M0 0
    x[3, :] = np.linspace(-3, 3, 128, dtype=np.float32)
    out, sc = oracle.quantize_rows(x)
    assert sc[0].tolist() == [0, 0, 0, 0] and not out[0].any()
    assert sc[1, 0] == 127 and out[1, 0] == 126 and sc[1, 1] == 127 and out[1, 32] == 126
    assert sc[2, 0] == 0
    tab = oracle.e4m3_table()
    deq = tab[out[3]].reshape(4, 32) * (2.0 ** (sc[3].astype(np.float64) - 127))[:, None]
    assert np.abs(deq.ravel() - x[3]).max() <= 2.0 ** -4 * 3.0      # e4m3 has 3 mantissa bits: half an ulp of 2^-3 relative


@pytest.mark.gpu
def test_device_quantisers_equal_the_oracle_bit_for_bit(oracle):
    torch = pytest.importorskip("torch")
    from amdgpu_rustdsl_b200 import Q_PRESCALE, quantize_qk, quantize_v
    rng = np.random.default_rng(7)
    for rows in (1, 3, 16, 1000, 65536 + 5):
        x = (rng.standard_normal((rows, 128)) * np.exp2(rng.integers(-12, 12, (rows, 1)))).astype(np.float32)
        x[0, :32] = 0.0
        if rows > 2:
            x[1, 5] = 3.0e38
            x[2, :] = 2.0 ** -130
        xb = torch.from_numpy(x).to(torch.bfloat16).cuda()
        xf = xb.float().cpu().numpy()                      # the bf16 values the device sees
        for mul in (1.0, Q_PRESCALE):
            out = torch.full((rows, 128), 0xAA, dtype=torch.uint8, device="cuda")
            sc = torch.full((rows * 4 + 64,), 0xAA, dtype=torch.uint8, device="cuda")
            quantize_qk(xb, out, sc, mul=mul)
            torch.cuda.synchronize()
            want, want_sc = oracle.quantize_rows(xf, np.float32(mul))
            assert np.array_equal(sc.cpu().numpy()[: rows * 4].reshape(rows, 4), want_sc), (rows, mul)
            assert np.array_equal(out.cpu().numpy(), want), (rows, mul)
            assert (sc.cpu().numpy()[rows * 4:] == 0xAA).all()      # nothing written past the rows
    for n in (8, 128 * 77, 128 * 4096 + 8):
        x = (rng.standard_normal(n) * 3.0).astype(np.float32)
        xb = torch.from_numpy(x).to(torch.bfloat16).cuda()
        out = torch.empty(n, dtype=torch.uint8, device="cuda")
        vd = torch.zeros(1024, dtype=torch.float32, device="cuda")
        quantize_v(xb, out, vd)
        torch.cuda.synchronize()
        want, want_vd = oracle.quantize_tensor(xb.float().cpu().numpy())
        assert float(vd[0]) == np.float32(want_vd) and np.array_equal(out.cpu().numpy(), want), n
    z = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    out = torch.full((64,), 0xAA, dtype=torch.uint8, device="cuda")
    vd = torch.zeros(2, dtype=torch.float32, device="cuda")
    quantize_v(z, out, vd)
    assert float(vd[0]) == 1.0 and not out.cpu().numpy().any()


@pytest.mark.gpu
def test_quantise_then_attend_passes_the_gate(oracle):
    """bf16 Q, K, V -> device quantisers -> attention, scored like every other shape: against the fp64 oracle on the quantised operands
    and the reference path's error on the same operands."""
    torch = pytest.importorskip("torch")
    from amdgpu_rustdsl_b200 import Q_PRESCALE, fmha_fwd_mxfp8, quantize_qk, quantize_v
    B, H, HK, S, SK = 1, 4, 2, 300, 1337
    g = torch.Generator().manual_seed(11)
    q = torch.randn(B, S, H, 128, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(B, SK, HK, 128, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(B, SK, HK, 128, generator=g).to(torch.bfloat16).cuda()
    q8, k8, v8 = (torch.empty(t.shape, dtype=torch.uint8, device="cuda") for t in (q, k, v))
    qs = torch.zeros(B * S * H * 4 + 512 * H * 4, dtype=torch.uint8, device="cuda")
    ks = torch.zeros(B * SK * HK * 4 + 640 * H * 4, dtype=torch.uint8, device="cuda")
    vs = torch.zeros(1024, dtype=torch.float32, device="cuda")
    quantize_qk(q, q8, qs, mul=Q_PRESCALE)
    quantize_qk(k, k8, ks)
    quantize_v(v, v8, vs)
    out = torch.full((B, S, H, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    fmha_fwd_mxfp8(q8, k8, v8, qs, ks, vs, out)
    torch.cuda.synchronize()
    inp = oracle.Inputs(B, H, HK, S, SK, q8.cpu().numpy(), k8.cpu().numpy(), v8.cpu().numpy(), qs.cpu().numpy(), ks.cpu().numpy(), float(vs[0]))
    rows = 32
    ref = oracle.reference(inp, rows)
    ours = oracle.compare(inp, out.view(torch.int16).cpu().numpy().view(np.uint16), ref, rows)
    theirs = oracle.compare(inp, oracle.recipe_forward(inp, rows, 0), ref, rows)
    assert ours.bad <= theirs.bad and ours.mean_err <= 1.10 * theirs.mean_err and ours.worst_err <= 2e-2, (ours, theirs)
    # and the quantised attention is close to plain bf16 attention on the unquantised tensors (a sanity bound, not a gate)
    qf, kf, vf = q.float(), k.float().repeat_interleave(H // HK, dim=2), v.float().repeat_interleave(H // HK, dim=2)
    s = torch.einsum("bshd,bthd->bhst", qf, kf) / 128 ** 0.5
    want = torch.einsum("bhst,bthd->bshd", torch.softmax(s, -1), vf)
    assert (out.float() - want).abs().max().item() < 0.05
