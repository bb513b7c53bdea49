"""CPU checks of the oracle: CPU ATen against the committed golden vectors and
against the independent plain-C restatement of the order-sensitive index
algorithms."""
import numpy as np
import torch

from oracle import aten_cpu, seq_ref


def test_reference_binary_cases_match_golden(golden):
    g = golden("ref_binary")
    for c in g["cases"]:
        fn = getattr(torch.ops.aten, c["op"])
        kw = {"alpha": c["alpha"]} if "alpha" in c else {}
        out = fn(c["lhs"], c["rhs"], **kw)
        assert out.dtype == c["out"].dtype and out.shape == c["out"].shape
        assert torch.isclose(out, c["out"], rtol=g["rtol"], atol=g["atol"]).all()


def test_reference_linear_cases_match_golden(golden):
    g = golden("ref_linear")
    assert torch.allclose(aten_cpu.addmm(g["addmm"]["c"], g["addmm"]["m1"], g["addmm"]["m2"]), g["addmm"]["out"])
    assert torch.allclose(aten_cpu.mm(g["mm"]["m1"], g["mm"]["m2"]), g["mm"]["out"])
    assert torch.allclose(aten_cpu.bmm(g["bmm"]["b1"], g["bmm"]["b2"]), g["bmm"]["out"])
    l = g["linear"]
    assert torch.allclose(torch.ops.aten.linear(l["x"], l["w"], l["b"]), l["out"])


def test_small_op_cases_match_golden(golden):
    g = golden("op_small")
    assert torch.equal(aten_cpu.silu(g["silu"]["a"]), g["silu"]["out"])
    assert torch.equal(aten_cpu.cast(g["cast"]["a"], torch.bfloat16), g["cast"]["bf16"])
    assert torch.allclose(aten_cpu.softmax(g["softmax"]["a"], -1), g["softmax"]["out"], rtol=1e-6, atol=1e-7)
    ln = g["layer_norm"]
    y, mean, rstd = aten_cpu.native_layer_norm(ln["a"], (130,), ln["w"], ln["b"], ln["eps"])
    assert torch.allclose(y, ln["y"], rtol=1e-6, atol=1e-6)
    assert torch.equal(aten_cpu.embedding(g["embedding"]["table"], g["embedding"]["ids"]), g["embedding"]["out"])
    assert torch.equal(aten_cpu.gather(g["gather"]["src"], 1, g["gather"]["idx"]), g["gather"]["out"])
    s = g["scatter_add"]
    assert torch.equal(aten_cpu.scatter_add(s["self"], 0, s["rows"][:, None].expand(-1, 12), s["src"]), s["out"])
    p = g["index_put"]
    assert torch.equal(aten_cpu.index_put(p["self"], [p["rows"]], p["src"], True), p["out_acc"])
    r = g["rms_norm_residual"]
    y, h = aten_cpu.rms_norm_residual(r["x"], r["res"], r["w"], r["eps"])
    assert torch.equal(y, r["y"]) and torch.equal(h, r["h"])
    assert torch.equal(aten_cpu.rope(g["rope"]["q"], g["rope"]["cos"], g["rope"]["sin"]), g["rope"]["out"])
    assert torch.equal(aten_cpu.swiglu(g["swiglu"]["gate"], g["swiglu"]["up"]), g["swiglu"]["out"])


def test_c_restatement_pins_aten_accumulation_order(golden):
    g = golden("op_small")
    s = g["scatter_add"]
    c = seq_ref.scatter_add_rows(s["self"].numpy(), s["rows"].numpy(), s["src"].numpy())
    assert np.array_equal(c, s["out"].numpy())
    f = g["scatter_add_full"]
    c = seq_ref.scatter_add_dim0(f["self"].numpy(), f["index"].numpy(), f["src"].numpy())
    assert np.array_equal(c, f["out"].numpy())
    p = g["index_put"]
    assert np.array_equal(seq_ref.scatter_add_rows(p["self"].numpy(), p["rows"].numpy(), p["src"].numpy()),
                          p["out_acc"].numpy())
    assert np.array_equal(seq_ref.index_put_rows(p["self"].numpy(), p["rows"].numpy(), p["src"].numpy()),
                          p["out_set"].numpy())


def test_c_restatement_larger_random():
    gen = torch.Generator().manual_seed(7)
    src = torch.randn(20000, 8, generator=gen)
    rows = torch.randint(0, 500, (20000,), generator=gen)
    base = torch.randn(500, 8, generator=gen)
    a = aten_cpu.scatter_add(base, 0, rows[:, None].expand(-1, 8), src)
    assert np.array_equal(a.numpy(), seq_ref.scatter_add_rows(base.numpy(), rows.numpy(), src.numpy()))
    b = aten_cpu.index_put(base, [rows], src, True)
    assert torch.equal(a, b)
    table = torch.randn(500, 8, generator=gen)
    assert np.array_equal(aten_cpu.index_select(table, 0, rows[:100]).numpy(),
                          seq_ref.gather_rows(table.numpy(), rows[:100].numpy()))
    gi = torch.randint(0, 8, (500, 8), generator=gen)
    assert np.array_equal(aten_cpu.gather(table, 1, gi).numpy(), seq_ref.gather_lastdim(table.numpy(), gi.numpy()))


def test_bf16_rounding_rule():
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(100000, generator=gen)
    x[:4] = torch.tensor([float("inf"), -float("inf"), 0.0, -0.0])
    x[4] = torch.tensor(1.0) + 2.0 ** -9  # tie: rounds to even
    bits = x.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(bits, seq_ref.f32_to_bf16_bits(x.numpy()))
    # NaN stays NaN; its payload is not part of the contract (ATen's own scalar
    # and vectorised CPU casts disagree on it).
    n = seq_ref.f32_to_bf16_bits(np.array([np.nan], dtype=np.float32))
    assert np.isnan(seq_ref.bf16_bits_to_f32(n))[0]


def test_sdpa_formula_oracle_is_pinned_to_aten_cpu_kernel():
    """The fp32 formula used as the attention oracle against ATen's own CPU kernel -- the one the
    reference backend's op check compares a device result with
    (torch_gcu/csrc/aten/GCUNativeFunctions.cpp:49-102): causal, grouped-query, fp32 and bf16."""
    g = torch.Generator().manual_seed(11)
    for (B, Hq, Hkv, S, D) in [(2, 8, 2, 160, 128), (1, 4, 4, 77, 64), (1, 6, 1, 300, 128)]:
        q, k, v = (torch.randn(B, h, S, D, generator=g) for h in (Hq, Hkv, Hkv))
        out, lse = aten_cpu.sdpa_causal(q, k, v)
        aten = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        assert torch.allclose(out, aten, rtol=1e-5, atol=1e-5)
        # the op the reference registers, with its logsumexp output
        G = Hq // Hkv
        res = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(
            q, k.repeat_interleave(G, 1), v.repeat_interleave(G, 1), 0.0, True)
        assert torch.allclose(out, res[0], rtol=1e-5, atol=1e-5)
        assert torch.allclose(lse, res[1], rtol=1e-5, atol=1e-5)
        qb, kb, vb = q.bfloat16(), k.bfloat16(), v.bfloat16()
        ob, _ = aten_cpu.sdpa_causal(qb, kb, vb)
        atb = torch.nn.functional.scaled_dot_product_attention(qb, kb, vb, is_causal=True, enable_gqa=True)
        assert torch.allclose(ob.float(), atb.float(), rtol=1.6e-2, atol=1e-2)
