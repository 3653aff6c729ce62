"""Shared helpers of the parity tests: golden fixtures, tolerances, GPU runners."""
import hashlib
import os

import numpy as np
import torch

from oracle import attention_oracle as oracle

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# tolerances of the build (floating point): forward output max-abs, gradients relative L2
TOL_O_MAX_ABS = 2e-3
TOL_GRAD_REL_L2 = 1e-2
# the reference's own bar against its fp16 math path (test.py:42-45)
TOL_REFERENCE_ATOL = 1e-2
TOL_LSE_MAX_ABS = 2e-3
# bf16 tensors (8 significant bits instead of 11): the output is rounded to bf16, whose spacing is
# 2^-7 = 7.8e-3 for |O| in [1, 2) and twice that in [2, 4), and P is rounded to bf16 before P V
TOL_O_MAX_ABS_BF16 = 1.6e-2
TOL_GRAD_REL_L2_BF16 = 1e-2


def golden_names():
    return sorted(f[:-4] for f in os.listdir(GOLDEN_DIR) if f.endswith(".npz"))


def load_golden(name):
    """Fixture -> dict with rebuilt inputs (checked against the stored SHA-256) and the
    reference math path's fp16 outputs."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    Z, N, H, D = (int(x) for x in z["shape"])
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, int(z["seed"]))
    h = hashlib.sha256()
    for t in (q, k, v, dout):
        h.update(t.numpy().tobytes())
    assert h.hexdigest() == str(z["input_sha256"]), "seeded inputs differ from the fixture's"
    return dict(q=q, k=k, v=v, dout=dout, causal=bool(z["causal"]), scale=float(z["sm_scale"]),
                out=torch.from_numpy(z["out"]), dq=torch.from_numpy(z["dq"]),
                dk=torch.from_numpy(z["dk"]), dv=torch.from_numpy(z["dv"]))


def gpu_fwd_bwd(q, k, v, dout, scale, causal, causal_shift=0, device="cuda"):
    """Forward + backward through the C ABI on the GPU; returns CPU tensors
    (out fp16, lse fp32, dq, dk, dv fp16) and checks the status word."""
    from flash_attn_v100 import cabi

    qd, kd, vd, dod = (t.to(device) for t in (q, k, v, dout))
    status = torch.zeros(1, dtype=torch.int32, device=device)
    out, lse = cabi.fwd(qd, kd, vd, scale, causal, causal_shift, status=status)
    dq, dk, dv = cabi.bwd(qd, kd, vd, out, dod, lse, scale, causal, causal_shift, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"kernel status word = {int(status.item()):#x}"
    return out.cpu(), lse.cpu(), dq.cpu(), dk.cpu(), dv.cpu()


def check_against_oracle(got, ref, what="", tol_o=TOL_O_MAX_ABS, tol_grad=TOL_GRAD_REL_L2):
    """got = (out, lse, dq, dk, dv) from the GPU; ref = the same from the oracle (fp32)."""
    out, lse, dq, dk, dv = got
    r_out, r_lse, r_dq, r_dk, r_dv = ref
    e_o = oracle.max_abs(out.float(), r_out)
    finite = torch.isfinite(r_lse)
    e_l = oracle.max_abs(lse[finite], r_lse[finite]) if finite.any() else 0.0
    assert torch.equal(torch.isfinite(lse), finite), f"{what}: LSE finiteness differs"
    e_dq, e_dk, e_dv = (oracle.rel_l2(a.float(), b) for a, b in ((dq, r_dq), (dk, r_dk), (dv, r_dv)))
    msg = f"{what}: O max-abs {e_o:.2e}, LSE {e_l:.2e}, rel-L2 dQ {e_dq:.2e} dK {e_dk:.2e} dV {e_dv:.2e}"
    print(msg)
    assert e_o <= tol_o, msg
    assert e_l <= TOL_LSE_MAX_ABS, msg
    assert e_dq <= tol_grad and e_dk <= tol_grad and e_dv <= tol_grad, msg
    return e_o, e_dq, e_dk, e_dv
