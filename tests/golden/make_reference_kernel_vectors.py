"""Makes ``reference_kernels.npz``: outputs of the reference's own float32 CUDA kernels
(src/cuda_kernels.cu of yusiwen/minfer: rms_norm_f32, rope_f32, swiglu_f32, gqa_attn_f32 with
store_kv_f32) on small seeded inputs, against which ``tests/test_plain.py`` checks the plain
implementation's functions.  The reference's model code is Rust and cannot be built here; its
CUDA kernels are plain C and can.

    nvcc -shared -Xcompiler -fPIC -gencode arch=compute_100a,code=sm_100a -O2 \\
         -o libref_kernels.so <reference>/src/cuda_kernels.cu
    python tests/golden/make_reference_kernel_vectors.py libref_kernels.so tests/golden/reference_kernels.npz

Needs a GPU.  The library is the reference's file compiled as it is; nothing of it is part
of this repository.  Inputs are regenerated from the seeds by the test, so only the outputs
are stored (float32)."""
import ctypes
import sys

import numpy as np
import torch


def inputs():
    """The cases, as float32 CPU tensors made from fixed seeds."""
    g = torch.Generator().manual_seed(2024)
    cases = {}
    cases["rms_norm"] = {"x": torch.randn(5, 72, generator=g) * 3.0,
                         "w": 1.0 + 0.2 * torch.randn(72, generator=g), "eps": 1e-6}
    cases["rope"] = {"x": torch.randn(6, 3, 16, generator=g), "positions": [0, 1, 2, 7, 300, 4095],
                     "theta": 1000000.0, "scale": 1.0}
    cases["rope_base_10000"] = {"x": torch.randn(4, 2, 64, generator=g), "positions": [3, 4, 5, 2000],
                                "theta": 10000.0, "scale": 1.0}
    cases["swiglu"] = {"gate": torch.randn(200, generator=g) * 4.0, "up": torch.randn(200, generator=g)}
    # attention: one sequence of 70 tokens at positions 0..69, 6 heads on 2 key/value heads of 32
    cases["attention"] = {"q": torch.randn(70, 6, 32, generator=g), "k": torch.randn(70, 2, 32, generator=g),
                          "v": torch.randn(70, 2, 32, generator=g), "scale": 1.0 / 32 ** 0.5}
    return cases


def main(lib_path: str, out_path: str) -> int:
    lib = ctypes.CDLL(lib_path)
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.launch_rms_norm_f32.argtypes = [vp, vp, vp, ci, cf, ci, vp]
    lib.launch_rope_f32.argtypes = [vp, ci, ci, ci, cf, cf, vp, vp]
    lib.launch_swiglu_f32.argtypes = [vp, vp, vp, ci, vp]
    lib.launch_store_kv_f32.argtypes = [vp, vp, ci, ci, vp, vp]
    lib.launch_gqa_attn_f32.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, cf, ci, vp]
    c = inputs()
    out = {}
    dev = "cuda:0"
    stream = None                                     # the default stream

    x, w = c["rms_norm"]["x"].to(dev), c["rms_norm"]["w"].to(dev)
    y = torch.empty_like(x)
    lib.launch_rms_norm_f32(x.data_ptr(), w.data_ptr(), y.data_ptr(), x.shape[1], c["rms_norm"]["eps"],
                            x.shape[0], stream)
    out["rms_norm"] = y.cpu().numpy()

    for name in ("rope", "rope_base_10000"):
        x = c[name]["x"].to(dev).clone()
        pos = torch.tensor(c[name]["positions"], dtype=torch.int32, device=dev)
        lib.launch_rope_f32(x.data_ptr(), x.shape[1], x.shape[2], x.shape[0], c[name]["theta"],
                            c[name]["scale"], pos.data_ptr(), stream)
        out[name] = x.cpu().numpy()

    gate, up = c["swiglu"]["gate"].to(dev), c["swiglu"]["up"].to(dev)
    dst = torch.empty_like(gate)
    lib.launch_swiglu_f32(gate.data_ptr(), up.data_ptr(), dst.data_ptr(), gate.numel(), stream)
    out["swiglu"] = dst.cpu().numpy()

    a = c["attention"]
    q, k, v = a["q"].to(dev), a["k"].to(dev), a["v"].to(dev)
    T, nh, hd = q.shape
    nk = k.shape[1]
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    kc = torch.zeros(128, nk * hd, device=dev)        # a cache of 128 positions
    vc = torch.zeros_like(kc)
    lib.launch_store_kv_f32(k.data_ptr(), kc.data_ptr(), nk * hd, T, pos.data_ptr(), stream)
    lib.launch_store_kv_f32(v.data_ptr(), vc.data_ptr(), nk * hd, T, pos.data_ptr(), stream)
    o = torch.empty_like(q)
    lib.launch_gqa_attn_f32(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), pos.data_ptr(),
                            nh, nk, hd, a["scale"], T, stream)
    torch.cuda.synchronize()
    out["attention"] = o.cpu().numpy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1], sys.argv[2]))
