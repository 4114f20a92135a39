"""Backward kernels (delta, dK/dV, dQ) against torch autograd through the fp32 oracle.
Tolerance (stated by the task): max-abs 5e-2 on dQ, dK, dV."""
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu
G_TOL = 5e-2


def _grads(q, k, v, do, mask, sm_scale):
    from fa2_custom_mask import flash_attention_custom_mask
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = flash_attention_custom_mask(qc, kc, vc, mask.cuda(), sm_scale)
    o.backward(do.cuda())
    torch.cuda.synchronize()
    return o.detach().float().cpu(), qc.grad.float().cpu(), kc.grad.float().cpu(), vc.grad.float().cpu()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,N,p,diag,causal", [
    (1, 1, 64, 1.0, True, False),
    (1, 1, 128, 1.0, True, False),
    (1, 2, 192, 0.5, True, False),
    (2, 2, 256, 0.5, False, False),     # empty rows and empty columns
    (1, 2, 1024, 0.1, True, False),
    (1, 1, 512, 1.0, True, False),
    (2, 2, 512, 0.25, True, True),      # block-causal sparse (BASELINE config 5 pattern)
])
def test_gradients_match_autograd(lib, dtype, B, H, N, p, diag, causal):
    q, k, v, do = oracle.make_qkv(B, H, N, 64, seed=N + H, dtype=dtype, n=4)
    mask = oracle.make_block_mask(B, H, N // 64, p, seed=N + 1, diagonal=diag, causal=causal)
    o, dq, dk, dv = _grads(q, k, v, do, mask, 0.125)
    o_ref, _, dq_ref, dk_ref, dv_ref = oracle.attn_forward_backward(q, k, v, mask, 0.125, do)
    assert (o - o_ref).abs().max() <= 2e-2
    for name, got, ref in (("dq", dq, dq_ref), ("dk", dk, dk_ref), ("dv", dv, dv_ref)):
        err = (got - ref).abs().max().item()
        assert err <= G_TOL, f"{name} max-abs err {err}"


def test_delta_kernel(lib):
    import ctypes
    from fa2_custom_mask import _lib
    o, do = (t.cuda() for t in oracle.make_qkv(2, 3, 320, 64, seed=1, dtype=torch.bfloat16, n=2))
    delta = torch.empty(2, 3, 320, dtype=torch.float32, device="cuda")
    _lib.check("bsa_attn_bwd_delta", lib.bsa_attn_bwd_delta(
        _lib.ptr(o), _lib.ptr(do), _lib.strides4(o), _lib.ptr(delta), _lib.BSA_BF16, 2, 3, 320, 64,
        _lib.stream_ptr()))
    ref = (o.float() * do.float()).sum(-1)
    assert (delta - ref).abs().max().item() <= 1e-4


def test_shared_mask_and_dense_mask_backward(lib):
    q, k, v, do = oracle.make_qkv(2, 2, 256, 64, seed=12, dtype=torch.float16, n=4)
    shared = oracle.make_block_mask(1, 1, 4, 0.5, seed=12)
    o, dq, dk, dv = _grads(q, k, v, do, shared, 0.125)
    ref = oracle.attn_forward_backward(q, k, v, shared.expand(2, 2, 4, 4), 0.125, do)
    for got, r in ((dq, ref[2]), (dk, ref[3]), (dv, ref[4])):
        assert (got - r).abs().max() <= G_TOL
    o2, dq2, dk2, dv2 = _grads(q, k, v, do, oracle.expand_block_mask(shared), 0.125)
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)


def test_baseline_config5_shape_one_head(lib):
    """One (batch, head) of BASELINE config 5 (N=16384, block-causal, p=0.25) against the fp32
    arithmetic evaluated on the GPU in chunks; autograd on the CPU would take minutes."""
    from fa2_custom_mask import flash_attention_custom_mask
    N = 16384
    q, k, v, do = (t.cuda() for t in oracle.make_qkv(1, 1, N, 64, seed=55, dtype=torch.bfloat16, n=4))
    mask = oracle.make_block_mask(1, 1, N // 64, 0.25, seed=55, causal=True).cuda()
    qc, kc, vc = (t.clone().requires_grad_(True) for t in (q, k, v))
    o = flash_attention_custom_mask(qc, kc, vc, mask, 0.125)
    o.backward(do)
    qf, kf, vf, dof = (t[0, 0].float() for t in (q, k, v, do))
    dk_ref = torch.zeros_like(kf)
    dv_ref = torch.zeros_like(vf)
    worst_dq = 0.0
    for r0 in range(0, N, 1024):
        r1 = r0 + 1024
        dense = mask[0, 0, r0 // 64:r1 // 64].repeat_interleave(64, 0).repeat_interleave(64, 1)
        s = (qf[r0:r1] @ kf.T) * 0.125
        p = torch.softmax(s.masked_fill(~dense, float("-inf")), -1)
        oc = p @ vf
        dp = dof[r0:r1] @ vf.T
        ds = p * (dp - (oc * dof[r0:r1]).sum(-1, keepdim=True))
        worst_dq = max(worst_dq, (qc.grad[0, 0, r0:r1].float() - 0.125 * ds @ kf).abs().max().item())
        dk_ref += 0.125 * ds.T @ qf[r0:r1]
        dv_ref += p.T @ dof[r0:r1]
    assert worst_dq <= G_TOL
    assert (kc.grad[0, 0].float() - dk_ref).abs().max().item() <= G_TOL
    assert (vc.grad[0, 0].float() - dv_ref).abs().max().item() <= G_TOL


def test_baseline_config5_shape_two_by_two_heads(lib):
    """B=2, H=2 of BASELINE config 5 (N=16384, block-causal, p=0.25, a different mask per head),
    with q, k, v and dO stored as [B,N,H,D] and viewed as [B,H,N,D]: forward and gradients of
    every (batch, head) against the fp32 arithmetic evaluated on the GPU in chunks."""
    from fa2_custom_mask import flash_attention_custom_mask
    B, H, N = 2, 2, 16384
    g = torch.Generator(device="cuda").manual_seed(56)
    q, k, v, do = (torch.randn(B, N, H, 64, device="cuda", generator=g).to(torch.bfloat16)
                   .transpose(1, 2) for _ in range(4))
    assert not q.is_contiguous()
    mask = oracle.make_block_mask(B, H, N // 64, 0.25, seed=56, causal=True).cuda()
    qc, kc, vc = (t.clone(memory_format=torch.preserve_format).requires_grad_(True)
                  for t in (q, k, v))
    o = flash_attention_custom_mask(qc, kc, vc, mask, 0.125)
    o.backward(do)
    for b in range(B):
        for h in range(H):
            qf, kf, vf, dof = (t[b, h].float() for t in (q, k, v, do))
            dk_ref = torch.zeros_like(kf)
            dv_ref = torch.zeros_like(vf)
            worst_o = worst_dq = 0.0
            for r0 in range(0, N, 2048):
                r1 = r0 + 2048
                dense = mask[b, h, r0 // 64:r1 // 64].repeat_interleave(64, 0).repeat_interleave(64, 1)
                s = (qf[r0:r1] @ kf.T) * 0.125
                p = torch.softmax(s.masked_fill(~dense, float("-inf")), -1)
                oc = p @ vf
                worst_o = max(worst_o, (o[b, h, r0:r1].float() - oc).abs().max().item())
                dp = dof[r0:r1] @ vf.T
                ds = p * (dp - (oc * dof[r0:r1]).sum(-1, keepdim=True))
                worst_dq = max(worst_dq,
                               (qc.grad[b, h, r0:r1].float() - 0.125 * ds @ kf).abs().max().item())
                dk_ref += 0.125 * ds.T @ qf[r0:r1]
                dv_ref += p.T @ dof[r0:r1]
            assert worst_o <= 2e-2 and worst_dq <= G_TOL, (b, h, worst_o, worst_dq)
            assert (kc.grad[b, h].float() - dk_ref).abs().max().item() <= G_TOL
            assert (vc.grad[b, h].float() - dv_ref).abs().max().item() <= G_TOL


@pytest.mark.parametrize("D", [16, 32])
def test_small_head_dimensions_are_padded(lib, D):
    """The reference accepts D in {16, 32, 64, 128, 256} (fa2_custom_mask.py:58); 16 and 32 run on
    the D = 64 kernels with zero columns appended."""
    q, k, v, do = oracle.make_qkv(1, 2, 256, D, seed=D, dtype=torch.float16, n=4)
    mask = oracle.make_block_mask(1, 2, 4, 0.5, seed=D)
    sm_scale = D ** -0.5
    o, dq, dk, dv = _grads(q, k, v, do, mask, sm_scale)
    assert o.shape == q.shape and dq.shape == q.shape and dv.shape == v.shape
    o_ref, _, dq_ref, dk_ref, dv_ref = oracle.attn_forward_backward(q, k, v, mask, sm_scale, do)
    assert (o - o_ref).abs().max() <= 2e-2
    for got, ref in ((dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
        assert (got - ref).abs().max().item() <= G_TOL


def test_large_head_dimensions_are_refused(lib):
    from fa2_custom_mask import flash_attention_custom_mask
    q = torch.zeros(1, 1, 64, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(NotImplementedError):
        flash_attention_custom_mask(q, q, q, None, 0.1)


def test_rows_on_16_byte_boundaries_only(lib):
    """Operands and gradients whose rows start on 16-byte but not 32-byte boundaries (row stride 72
    elements, first row 8 elements in): the narrow store path of the write-out gives the same bits as
    the whole-sector stores used for aligned rows."""
    from fa2_custom_mask import attention_backward, attention_forward, build_tile_lists
    B, H, N = 1, 2, 256
    q, k, v, do = (t.cuda() for t in oracle.make_qkv(B, H, N, 64, seed=21, dtype=torch.bfloat16, n=4))
    mask = oracle.make_block_mask(B, H, N // 64, 0.6, seed=5).cuda()
    lists = build_tile_lists(mask)
    o, lse2, _ = attention_forward(q, k, v, lists, 0.125)
    ref = attention_backward(q, k, v, o, lse2, do, lists, 0.125)

    def shifted(t):
        wide = torch.zeros(B, H, N, 72, dtype=t.dtype, device="cuda")
        view = wide[..., 8:]
        view.copy_(t)
        assert view.data_ptr() % 32 == 16 and view.stride(2) == 72
        return view
    qs, ks, vs, os_, dos = (shifted(t) for t in (q, k, v, o, do))
    got = attention_backward(qs, ks, vs, os_, lse2, dos, lists, 0.125)
    torch.cuda.synchronize()
    for g, r in zip(got, ref):
        assert g.stride() == qs.stride() or g.is_contiguous()
        assert torch.equal(g.float(), r.float())


def test_forward_and_backward_in_a_graph(lib):
    """A whole training step of the public op (mask reduction, forward, tile lists, delta, dK/dV,
    dQ) holds no host synchronisation: it is captured into a CUDA graph and replayed on new inputs
    (mask included) written into the same buffers."""
    from fa2_custom_mask import flash_attention_custom_mask
    B, H, N = 1, 2, 512
    q, k, v, do = (t.cuda() for t in oracle.make_qkv(B, H, N, 64, seed=31, dtype=torch.bfloat16, n=4))
    block = oracle.make_block_mask(B, H, N // 64, 0.4, seed=31).cuda()
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(2):   # loads the library and warms the allocator outside the capture
            flash_attention_custom_mask(q, k, v, block, 0.125).backward(do)
        torch.cuda.synchronize()
        q.grad = k.grad = v.grad = None
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            out = flash_attention_custom_mask(q, k, v, block, 0.125)
            out.backward(do)
        for seed in (32, 33):
            q2, k2, v2, do2 = oracle.make_qkv(B, H, N, 64, seed=seed, dtype=torch.bfloat16, n=4)
            block2 = oracle.make_block_mask(B, H, N // 64, 0.5, seed=seed)
            with torch.no_grad():
                q.copy_(q2); k.copy_(k2); v.copy_(v2); do.copy_(do2); block.copy_(block2)
            graph.replay()
            torch.cuda.synchronize()
            o_ref, _, dq_ref, dk_ref, dv_ref = oracle.attn_forward_backward(q2, k2, v2, block2, 0.125, do2)
            assert (out.detach().float().cpu() - o_ref).abs().max() <= 2e-2
            for got, ref in ((q.grad, dq_ref), (k.grad, dk_ref), (v.grad, dv_ref)):
                assert (got.float().cpu() - ref).abs().max() <= G_TOL
