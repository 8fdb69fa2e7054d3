"""The quantised Qwen3 model and the serving engine on a GPU (tiny random-init model)."""
import pytest
import torch

import nanoquantization_b200 as nq
from nanoquantization_b200.engine import LLMEngine
from nanoquantization_b200.models import Qwen3QuantizedForCausalLM

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tiny(dtype=torch.float16, seed=0):
    torch.manual_seed(seed)
    m = Qwen3QuantizedForCausalLM(2, 512, 256, 4, 2, 1024, 512, 4, 128, 64, False, 1e6, 1e-6, device=DEV, dtype=dtype)
    g = torch.Generator(device=DEV); g.manual_seed(seed)
    for mod in m.modules():
        if isinstance(mod, nq.WQLinear_GEMM):
            mod.qweight.copy_(torch.randint(-2 ** 31, 2 ** 31, mod.qweight.shape, generator=g, device=DEV, dtype=torch.int64).to(torch.int32))
            mod.qzeros.copy_(torch.randint(-2 ** 31, 2 ** 31, mod.qzeros.shape, generator=g, device=DEV, dtype=torch.int64).to(torch.int32))
            mod.qscales.copy_((torch.rand(mod.qscales.shape, generator=g, device=DEV) * 9e-3 + 1e-3).to(dtype))
    return m


def test_state_dict_keys_match_reference_names():
    m = _tiny()
    keys = set(m.state_dict().keys())
    for k in ("model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.qweight", "model.layers.0.self_attn.k_proj.qscales",
              "model.layers.1.self_attn.o_proj.qzeros", "model.layers.0.self_attn.q_norm.weight",
              "model.layers.0.mlp.gate_proj.qweight", "model.layers.1.mlp.down_proj.qscales",
              "model.layers.0.input_layernorm.weight", "model.layers.1.post_attention_layernorm.weight",
              "model.norm.weight", "lm_head.weight", "lm_head.bias"):
        assert k in keys, k


@torch.no_grad()
def test_fused_projections_give_the_same_hidden_states():
    m = _tiny()
    x = torch.randint(0, 512, (2, 24), device=DEV)
    pos = torch.arange(24, device=DEV).unsqueeze(0)
    h0 = m(x, pos)
    m.fuse_projections()
    h1 = m(x, pos)
    assert torch.isfinite(h0).all()
    assert float((h0.float() - h1.float()).abs().max()) <= 2e-2 * float(h0.float().abs().max())


@torch.no_grad()
def test_engine_first_token_matches_full_forward_and_graphs_match_eager():
    m = _tiny(seed=1)
    m.fuse_projections()
    prompts = [torch.randint(0, 512, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (5, 33, 17)]
    # the reference-style path: full-sequence forward, arg-max of the last position
    firsts = []
    for p in prompts:
        x = torch.tensor([p], device=DEV)
        h = m(x, torch.arange(len(p), device=DEV).unsqueeze(0))
        firsts.append(int(m.greedy_tokens(h[0, -1:])[0]))
    eager = LLMEngine(m, num_blocks=32, block_size=16, use_cuda_graph=False).generate(prompts, 6)
    graph = LLMEngine(m, num_blocks=32, block_size=16, use_cuda_graph=True).generate(prompts, 6)
    assert [o[0] for o in eager] == firsts
    assert eager == graph
    assert all(len(o) == 6 for o in eager)


def test_engine_continuous_batching_ragged_lengths():
    m = _tiny(seed=2)
    eng = LLMEngine(m, num_blocks=24, block_size=16, max_batch=3)
    prompts = [[1 + i] * (4 + 3 * i) for i in range(5)]
    outs = eng.generate(prompts, [2, 5, 3, 1, 4])
    assert [len(o) for o in outs] == [2, 5, 3, 1, 4]
    assert len(eng.blocks.free) == 24          # every block returned


# ------------------------------------------------------------ fused elementwise kernels
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@torch.no_grad()
def test_fused_kernels_match_reference_modules(dtype):
    from nanoquantization_b200.layers import fused
    from nanoquantization_b200.models import RMSNorm, RotaryCache
    g = torch.Generator(device=DEV).manual_seed(3)
    T, H, Hq, Hkv, D, I = 7, 1024, 4, 2, 128, 768
    ulp = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7

    def close(a, b):
        return float((a.float() - b.float()).abs().max()) <= 2 * ulp * max(1.0, float(b.float().abs().max()))

    x = torch.randn(T, H, generator=g, device=DEV).to(dtype)
    r = torch.randn(T, H, generator=g, device=DEV).to(dtype)
    norm = RMSNorm(H, 1e-6).to(DEV)
    norm.weight.data = (torch.rand(H, generator=g, device=DEV) + 0.5).to(dtype)
    out, res = fused.add_rmsnorm(x, r.clone(), norm.weight, 1e-6)
    assert torch.equal(res, x + r) and close(out, norm(x + r))
    out0, res0 = fused.add_rmsnorm(x, None, norm.weight, 1e-6)
    assert res0 is x and close(out0, norm(x))

    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, generator=g, device=DEV).to(dtype)
    qn, kn = RMSNorm(D, 1e-6).to(DEV), RMSNorm(D, 1e-6).to(DEV)
    qn.weight.data = (torch.rand(D, generator=g, device=DEV) + 0.5).to(dtype)
    kn.weight.data = (torch.rand(D, generator=g, device=DEV) + 0.5).to(dtype)
    rope = RotaryCache(D, 4096, 1e6).to(DEV)
    pos = torch.tensor([0, 1, 5, 100, 1000, 4095, 17], device=DEV)
    q_ref = qn(qkv[:, :Hq * D].reshape(T, Hq, D))
    k_ref = kn(qkv[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D))
    q_ref, k_ref = rope(q_ref, k_ref, pos)
    v_ref = qkv[:, (Hq + Hkv) * D:].clone()
    fused.qknorm_rope_(qkv, qn.weight, kn.weight, rope.cos_sin_cache, pos, Hq, Hkv, D, 1e-6)
    assert close(qkv[:, :Hq * D].reshape(T, Hq, D), q_ref)
    assert close(qkv[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D), k_ref)
    assert torch.equal(qkv[:, (Hq + Hkv) * D:], v_ref)

    gu = torch.randn(T, 2 * I, generator=g, device=DEV).to(dtype)
    assert close(fused.silu_mul(gu), torch.nn.functional.silu(gu[:, :I]) * gu[:, I:])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@torch.no_grad()
def test_qknorm_rope_stores_k_and_v_in_the_paged_cache(dtype):
    """The cache rows written by the fused launch equal the in-place result scattered with index_copy_."""
    from nanoquantization_b200.layers import fused
    from nanoquantization_b200.models import RotaryCache
    g = torch.Generator(device=DEV).manual_seed(9)
    T, Hq, Hkv, D, blocks, bs = 5, 4, 2, 128, 6, 16
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, generator=g, device=DEV).to(dtype)
    qw = (torch.rand(D, generator=g, device=DEV) + 0.5).to(dtype)
    kw = (torch.rand(D, generator=g, device=DEV) + 0.5).to(dtype)
    rope = RotaryCache(D, 4096, 1e6).to(DEV)
    pos = torch.tensor([3, 0, 77, 4095, 12], device=DEV)
    slots = torch.tensor([17, 0, 95, 33, 64], device=DEV)
    plain = qkv.clone()
    fused.qknorm_rope_(plain, qw, kw, rope.cos_sin_cache, pos, Hq, Hkv, D, 1e-6)
    kc = torch.full((blocks, bs, Hkv, D), 7.0, dtype=dtype, device=DEV)
    vc = torch.full((blocks, bs, Hkv, D), 7.0, dtype=dtype, device=DEV)
    fused.qknorm_rope_(qkv, qw, kw, rope.cos_sin_cache, pos, Hq, Hkv, D, 1e-6, (kc, vc, slots))
    assert torch.equal(qkv, plain)
    want_k = torch.full_like(kc, 7.0).view(-1, Hkv, D).index_copy_(0, slots, plain[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D))
    want_v = torch.full_like(vc, 7.0).view(-1, Hkv, D).index_copy_(0, slots, plain[:, (Hq + Hkv) * D:].reshape(T, Hkv, D))
    assert torch.equal(kc.view(-1, Hkv, D), want_k) and torch.equal(vc.view(-1, Hkv, D), want_v)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("K,I,M", [(2048, 6144, 1), (2048, 6144, 16), (1024, 1536, 4), (5120, 3200, 3), (256, 512, 2), (4096, 1024, 64)])
@torch.no_grad()
def test_gate_up_with_fused_activation_is_bit_identical_to_the_separate_steps(K, I, M, dtype):
    """forward_silu_mul == silu_mul(forward(x)) bit for bit, on shapes that take the fused epilogue
    (decode sizes, I a multiple of 512, K split across CTAs) and on shapes that fall back."""
    from nanoquantization_b200.layers import fused
    import oracle.awq_oracle as O
    host = O.make_case(K, 2 * I, M, group_size=128, dtype=dtype, seed=21, bias=(M == 4))
    lin = nq.WQLinear_GEMM(4, 128, K, 2 * I, DEV, host["bias"] is not None, dtype)
    lin.qweight.copy_(host["qweight"]); lin.qscales.copy_(host["qscales"]); lin.qzeros.copy_(host["qzeros"])
    if host["bias"] is not None:
        lin.bias.copy_(host["bias"])
    x = host["x"].to(DEV)
    want = fused.silu_mul(lin(x))
    got = lin.forward_silu_mul(x)
    assert got.shape == (M, I) and torch.equal(got, want)
    assert torch.equal(lin.forward_silu_mul(x), want)  # and again: the workspace is left reusable


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M", [1, 5, 16])
@torch.no_grad()
def test_linears_with_norm_prologue_and_residual_epilogue(M, dtype):
    """o_proj-like linear with the residual add inside (bit-identical to linear + add, and its sums of
    squares), then a q/k/v-like linear that takes the RMSNorm of that stream inside (same roundings as
    the separate norm; the mean of squares is added in a different order, hence a tolerance)."""
    from nanoquantization_b200.layers import fused
    import oracle.awq_oracle as O
    H, Kin, Nout = 1024, 2048, 1536
    a = O.make_case(Kin, H, M, group_size=128, dtype=dtype, seed=31)
    b = O.make_case(H, Nout, M, group_size=128, dtype=dtype, seed=32)
    lin_o = nq.WQLinear_GEMM(4, 128, Kin, H, DEV, False, dtype)
    lin_q = nq.WQLinear_GEMM(4, 128, H, Nout, DEV, False, dtype)
    for lin, c in ((lin_o, a), (lin_q, b)):
        lin.qweight.copy_(c["qweight"]); lin.qscales.copy_(c["qscales"]); lin.qzeros.copy_(c["qzeros"])
    g = torch.Generator(device=DEV).manual_seed(4)
    x = a["x"].to(DEV)
    res = torch.randn(M, H, generator=g, device=DEV).to(dtype)
    w = (torch.rand(H, generator=g, device=DEV) + 0.5).to(dtype)
    assert lin_o.fused_supported(M, residual=True) and lin_q.fused_supported(M, norm=True)
    h, ssq = lin_o.forward_fused(x, residual=res)
    assert torch.equal(h, lin_o(x) + res)
    from nanoquantization_b200 import _lib
    assert ssq.shape == (M, H // _lib.load().nqb200_decode_tile_columns())
    want_ss = (h.float() ** 2).sum(1)
    assert float((ssq.sum(1) - want_ss).abs().max()) <= 1e-5 * float(want_ss.max())
    got = lin_q.forward_fused(h, norm=(ssq, w, 1e-6))
    want = lin_q(fused.add_rmsnorm(h, None, w, 1e-6)[0])
    assert O.rel_err(got, want) <= 2e-3
    # and both at once on one linear, twice (the workspace stays reusable)
    for _ in range(2):
        h2, ssq2 = lin_o.forward_fused(x, residual=res)
        assert torch.equal(h2, h) and torch.equal(ssq2, ssq)


@pytest.mark.parametrize("dtype,M", [(torch.bfloat16, 16), (torch.float16, 7)])
@torch.no_grad()
def test_fused_decode_block_vs_oracle(dtype, M):
    """o_proj with the residual add inside, then a merged gate|up linear that takes the RMSNorm of that
    stream and applies silu(gate) * up, against the CPU oracle's arithmetic for the same steps."""
    import oracle.awq_oracle as O
    H, I, Kin = 1024, 1536, 2048
    a = O.make_case(Kin, H, M, dtype=dtype, seed=41)
    b = O.make_case(H, 2 * I, M, dtype=dtype, seed=42)
    lin_o = nq.WQLinear_GEMM(4, 128, Kin, H, DEV, False, dtype)
    lin_gu = nq.WQLinear_GEMM(4, 128, H, 2 * I, DEV, False, dtype)
    for lin, c in ((lin_o, a), (lin_gu, b)):
        lin.qweight.copy_(c["qweight"]); lin.qscales.copy_(c["qscales"]); lin.qzeros.copy_(c["qzeros"])
    assert lin_o.fused_supported(M, residual=True) and lin_gu.fused_supported(M, norm=True, silu_mul=True)
    g = torch.Generator().manual_seed(5)
    res = torch.randn(M, H, generator=g).to(dtype)
    w = (torch.rand(H, generator=g) + 0.5).to(dtype)
    h, ssq = lin_o.forward_fused(a["x"].to(DEV), residual=res.to(DEV))
    y = lin_gu.forward_fused(h, norm=(ssq, w.to(DEV), 1e-6), silu_mul=True)
    torch.cuda.synchronize()
    tol = 2e-3 if dtype == torch.float16 else 8e-3
    y_o = O.w4a16_ref(a["x"], a["qweight"], a["qscales"], a["qzeros"]).to(dtype)
    h_ref = y_o + res
    assert O.rel_err(h, h_ref) <= tol
    hf = h_ref.float()
    xn = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(dtype) * w
    gu = O.w4a16_ref(xn, b["qweight"], b["qscales"], b["qzeros"]).to(dtype)
    want = (torch.nn.functional.silu(gu[:, :I]).to(dtype) * gu[:, I:]).float()
    assert O.rel_err(y, want) <= 2 * tol   # three 16-bit roundings (y, silu, product) on top of the GEMM's
