"""Forward parity against the reference's own Triton kernel run on the same GPU.

The reference package cannot be imported next to this one (both are called fa2_custom_mask), so it
runs in a child process from a copy under baseline/_ref (not part of the repository's history).
Skipped when that copy or Triton is missing; a copy that is there but does not run is a failure.
Tolerance (stated by the task): max-abs 2e-2 on O."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
O_TOL = 2e-2

CHILD = r"""
import sys, numpy as np, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2])
from oracle import oracle
from fa2_custom_mask.fa2_custom_mask import build_groups_from_block_mask
from fa2_custom_mask.fa2_fwd import _attn_fwd
B, H, N, p, seed, dt, out = int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5]), float(sys.argv[6]), int(sys.argv[7]), sys.argv[8], sys.argv[9]
dtype = torch.float16 if dt == "f16" else torch.bfloat16
q, k, v = (t.cuda() for t in oracle.make_qkv(B, H, N, 64, seed=seed, dtype=dtype))
mask = oracle.make_block_mask(B, H, N // 64, p, seed=seed).cuda()
groups, nlist = build_groups_from_block_mask(mask)
o = torch.zeros_like(q)
M = torch.full((B, H, N), float("nan"), device="cuda", dtype=torch.float32)
_attn_fwd[(groups.shape[0],)](q, k, v, groups, nlist, 0.125, M, o, *q.stride(), *k.stride(),
                               *v.stride(), *o.stride(), B, H, N, HEAD_DIM=64)
torch.cuda.synchronize()
np.savez(out, o=o.float().cpu().numpy(), M=M.cpu().numpy())
"""


def _reference_available():
    if not os.path.exists(os.path.join(REF_DIR, "fa2_custom_mask", "fa2_fwd.py")):
        return False
    try:
        import triton  # noqa: F401
    except Exception:
        return False
    return True


@pytest.mark.skipif(not _reference_available(), reason="no copy of the reference, or no Triton")
@pytest.mark.parametrize("B,H,N,p,dt", [(1, 2, 1024, 0.3, "f16"), (2, 2, 512, 1.0, "f16"),
                                        (1, 1, 2048, 0.1, "bf16")])
def test_forward_matches_the_reference_kernel_on_this_gpu(lib, tmp_path, B, H, N, p, dt):
    from fa2_custom_mask import attention_forward_masked
    out = str(tmp_path / "ref.npz")
    seed = N + H
    proc = subprocess.run([sys.executable, "-c", CHILD, REF_DIR, ROOT, str(B), str(H), str(N),
                           str(p), str(seed), dt, out], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, "the reference kernel did not run here: " + proc.stderr.strip()[-600:]
    ref = np.load(out)
    dtype = torch.float16 if dt == "f16" else torch.bfloat16
    q, k, v = (t.cuda() for t in oracle.make_qkv(B, H, N, 64, seed=seed, dtype=dtype))
    mask = oracle.make_block_mask(B, H, N // 64, p, seed=seed).cuda()
    o, lse2, rowmax = attention_forward_masked(q, k, v, mask, 0.125, want_rowmax=True)
    o_ref = torch.from_numpy(ref["o"])
    m_ref = torch.from_numpy(ref["M"])
    written = ~torch.isnan(m_ref)
    assert written.all()                     # the diagonal keeps every row non-empty
    assert (o.float().cpu() - o_ref).abs().max().item() <= O_TOL
    # the reference's M is the running row maximum in the exp2 domain
    assert (rowmax.cpu() - m_ref).abs().max().item() <= 2e-2
