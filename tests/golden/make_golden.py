"""Generate the golden fixtures in this directory from the REFERENCE'S OWN math path.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py [/path/to/flash-attention-v100]

The reference has no importable CPU implementation and no golden vectors; the code its test
compares the kernel against is the block of statements ``test.py:13-26`` (torch math path:
fp16 matmul, tril mask, fp32 softmax cast back to fp16, fp16 matmul, autograd backward).  This
script reads those statements from the reference's ``test.py`` as text, changes nothing but the
device string (``"cuda"`` -> ``"cpu"``), and executes them on seeded CPU inputs for each case
below.  The outputs (fp16 out, dq, dk, dv, exactly what the reference's asserts at
``test.py:42-45`` compare against) are stored as ``<case>.npz`` together with a SHA-256 of the
input bytes, so that tests can rebuild the inputs from the seed and prove they are the same.

Nothing at test time reads the reference checkout: the fixtures are self-contained.
"""
import hashlib
import os
import sys
import textwrap

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle.attention_oracle import make_inputs  # noqa: E402

# name: (Z, N, H, D, causal, sm_scale, seed)
CASES = {
    # BASELINE config 1: the CPU-runnable reference case
    "cfg1_z2_h4_n128_d64_noncausal": (2, 128, 4, 64, False, 1.0 / 8.0, 0),
    "z1_h2_n128_d64_causal": (1, 128, 2, 64, True, 1.0 / 8.0, 1),
    # the reference test's own settings (causal, sm_scale = 0.1, seed 20, D = 128), shrunk
    "z1_h2_n96_d128_causal_s01": (1, 96, 2, 128, True, 0.1, 20),
    "z1_h1_n160_d128_noncausal": (1, 160, 1, 128, False, 128 ** -0.5, 3),
}


def reference_math_path_source(ref_root: str) -> str:
    with open(os.path.join(ref_root, "test.py")) as f:
        lines = f.read().splitlines()
    block = "\n".join(lines[12:26])  # test.py:13-26, the body of `for i in range(1):`
    block = textwrap.dedent(block).replace('device="cuda"', 'device="cpu"')
    assert "torch.softmax(p.float(), dim=-1).half()" in block, "reference test.py changed?"
    return block


def input_digest(q, k, v, dout) -> str:
    h = hashlib.sha256()
    for t in (q, k, v, dout):
        h.update(t.numpy().tobytes())
    return h.hexdigest()


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to a checkout of flash-attention-v100>")
    ref_root = sys.argv[1]
    src = reference_math_path_source(ref_root)
    for name, (Z, N, H, D, causal, sm_scale, seed) in CASES.items():
        q, k, v, dout = make_inputs(Z, N, H, D, seed)
        digest = input_digest(q, k, v, dout)
        q.requires_grad_()
        k.requires_grad_()
        v.requires_grad_()
        ns = dict(torch=torch, q=q, k=k, v=v, dout=dout, sm_scale=sm_scale, causal=causal,
                  N_CTX=N, Z=Z, H=H, D_HEAD=D)
        exec(src, ns)  # the reference's statements, verbatim
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            out=ns["ref_out"].detach().numpy(), dq=ns["ref_dq"].numpy(), dk=ns["ref_dk"].numpy(),
            dv=ns["ref_dv"].numpy(), shape=np.array([Z, N, H, D]), causal=np.array(causal),
            sm_scale=np.array(sm_scale, dtype=np.float64), seed=np.array(seed),
            input_sha256=np.array(digest))
        print(name, "ok", digest[:12])


if __name__ == "__main__":
    main()
