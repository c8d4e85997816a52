"""Generate the golden vectors under tests/golden/ from the REFERENCE's own oracle.

Run in a container where the reference project is mounted:

    python tests/golden/make_golden.py /path/to/reference

It loads `fast_diffusion_attention/reference.py` of the reference by file path (importing the package
itself needs the compiled sm90 extension), evaluates `attention_ref` / `attention_varlen_ref` in float32 on
seeded inputs, takes the gradients with `torch.autograd.grad`, and stores inputs-by-seed + outputs as
float32 arrays. Mask fixtures store the packed visibility matrices of `diffusion_mask`. The reference is only
needed to regenerate; the tests read the .npz files.
"""

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    path = os.path.join(root, "fast_diffusion_attention", "reference.py")
    spec = importlib.util.spec_from_file_location("fda_reference_original", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


# name -> (B, n, H, Hk, d, block_size, softcap, scale, dtype)
DENSE_CASES = {
    "c1_cpu_config": (2, 256, 4, 4, 64, 64, 0.0, None, "float32"),
    "odd_n_small_bs": (2, 37, 4, 2, 32, 3, 0.0, None, "float32"),
    "bs_gt_n": (1, 50, 2, 1, 16, 64, 0.0, 0.3, "float32"),
    "softcap": (1, 96, 4, 2, 64, 16, 15.0, None, "float32"),
    "n1": (1, 1, 2, 2, 8, 1, 0.0, None, "float32"),
    "bf16_gqa": (1, 130, 6, 2, 32, 32, 0.0, None, "bfloat16"),
}
VARLEN_CASES = {
    "varlen_mixed": ([17, 30, 1, 64, 0, 5], 4, 2, 32, 4, 0.0, "float32"),
    "varlen_softcap": ([40, 8, 33], 2, 2, 16, 13, 30.0, "float32"),
}
ROW_STRIDE = 8
MASK_CASES = [(n, bs) for n in (1, 2, 5, 16, 33, 100) for bs in (1, 2, 3, 4, 7, 16, 200)]


def make_inputs(seed, shape_q, shape_kv, dtype):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(shape_q, generator=g).to(dtype)
    k = torch.randn(shape_kv, generator=g).to(dtype)
    v = torch.randn(shape_kv, generator=g).to(dtype)
    do = torch.randn(shape_q, generator=g).to(dtype)
    return q, k, v, do


def main(root):
    ref = load_reference(root)
    torch.manual_seed(0)
    out = {}
    for idx, (name, (B, n, H, Hk, d, bs, cap, scale, dt)) in enumerate(DENSE_CASES.items()):
        dtype = getattr(torch, dt)
        q, k, v, do = make_inputs(1000 + idx, (B, 2 * n, H, d), (B, 2 * n, Hk, d), dtype)
        q, k, v = (t.requires_grad_() for t in (q, k, v))
        o, lse = ref.attention_ref(q, k, v, bs, softmax_scale=scale, softcap=cap)
        dq, dk, dv = torch.autograd.grad(o, (q, k, v), do)
        o_pt, lse_pt = ref.attention_ref(q, k, v, bs, softmax_scale=scale, softcap=cap, upcast=False,
                                         reorder_ops=True)
        # gradients of the same-precision evaluation: what the reference's tests take as "plain PyTorch" for dq, dk, dv
        # (tests/test_diffusion_attn.py:85-104 there: autograd through attention_ref(upcast=False, reorder_ops=True))
        dq_pt, dk_pt, dv_pt = torch.autograd.grad(o_pt, (q, k, v), do)
        rec = dict(seed=1000 + idx, out=o, lse=lse, dq=dq, dk=dk, dv=dv, out_pt=o_pt, lse_pt=lse_pt,
                   dq_pt=dq_pt, dk_pt=dk_pt, dv_pt=dv_pt)
        strided = ("out", "dq", "dk", "dv", "out_pt", "dq_pt", "dk_pt", "dv_pt")
        if name == "c1_cpu_config":
            # keep the fixture small: every ROW_STRIDE-th sequence position of the largest case
            rec = {key: (val[:, ::ROW_STRIDE] if key in strided else val) for key, val in rec.items()}
        out[name] = rec
    for idx, (name, (ns, H, Hk, d, bs, cap, dt)) in enumerate(VARLEN_CASES.items()):
        dtype = getattr(torch, dt)
        total = 2 * sum(ns)
        cu = torch.tensor([0] + list(np.cumsum([2 * x for x in ns])), dtype=torch.int32)
        q, k, v, do = make_inputs(2000 + idx, (total, H, d), (total, Hk, d), dtype)
        q, k, v = (t.requires_grad_() for t in (q, k, v))
        # the reference's varlen wrapper cannot take empty samples (logsumexp over 0 keys): drop them, the
        # packed result is unchanged because an empty sample contributes no rows
        cu_nz = torch.tensor(sorted(set(cu.tolist())), dtype=torch.int32)
        o, lse = ref.attention_varlen_ref(q, k, v, cu_nz, bs, softcap=cap)
        dq, dk, dv = torch.autograd.grad(o, (q, k, v), do)
        out[name] = dict(seed=2000 + idx, out=o, lse=lse, dq=dq, dk=dk, dv=dv)
    arrays = {}
    for name, d_ in out.items():
        for key, val in d_.items():
            arrays[f"{name}/{key}"] = (np.asarray(val) if not torch.is_tensor(val)
                                       else val.detach().float().numpy())
    np.savez_compressed(os.path.join(HERE, "attention_golden.npz"), **arrays)

    masks = {}
    for n, bs in MASK_CASES:
        m = ref.diffusion_mask(n, bs)
        masks[f"mask/{n}/{bs}"] = np.packbits(m.numpy())
        masks[f"pairs/{n}/{bs}"] = np.asarray(ref.num_visible_pairs(n, bs))
    np.savez_compressed(os.path.join(HERE, "mask_golden.npz"), **masks)
    print("wrote", len(arrays), "attention arrays and", len(masks), "mask arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <reference project root>")
    main(sys.argv[1])
