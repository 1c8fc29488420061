"""Makes ``reference_kernels.npz``: outputs of the reference's own float32 CUDA kernels
(src/cuda_kernels.cu of yusiwen/minfer: rms_norm_f32, rope_f32, swiglu_f32, gqa_attn_f32 with
store_kv_f32, add_bias_f32, add_f32) on small seeded inputs, against which
``tests/test_plain.py`` checks the plain implementation's functions, and one whole layer
chained through those launchers in the order of the reference's graph
(src/models/qwen2/graph.rs:63-176: norm, projections, bias, rotation of q and k, cache store,
attention, output projection, residual, norm, SwiGLU, residual; the matrix products, which the
reference does with quantized kernels, are float64 products on the host), against which it
checks the plain model's composition.  The reference's model code is Rust and cannot be built here; its
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
    cases["layer"] = layer_case(g)
    return cases


LAYER = {"hidden": 64, "heads": 4, "kv_heads": 2, "head_dim": 16, "ffn": 96, "tokens": 20,
         "theta": 10000.0, "eps": 1e-6}


def layer_case(g):
    """One layer's weights and input rows (float32, seeded)."""
    c = LAYER
    ne, nh, nk, hd, nf, T = c["hidden"], c["heads"], c["kv_heads"], c["head_dim"], c["ffn"], c["tokens"]

    def r(*shape, std=0.3):
        return torch.randn(*shape, generator=g) * std
    return {"h0": r(T, ne, std=1.0), "ln1": 1.0 + r(ne, std=0.1), "ln2": 1.0 + r(ne, std=0.1),
            "final": 1.0 + r(ne, std=0.1),
            "wq": r(nh * hd, ne), "bq": r(nh * hd), "wk": r(nk * hd, ne), "bk": r(nk * hd),
            "wv": r(nk * hd, ne), "bv": r(nk * hd), "wo": r(ne, nh * hd),
            "wg": r(nf, ne), "wu": r(nf, ne), "wd": r(ne, nf)}


def host_product(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x W^T in float64 on the host, rounded once to float32 (the same on every machine)."""
    return (x.double().cpu() @ w.double().cpu().t()).float()


def run_layer(lib, c, dev, stream):
    """The layer through the reference's launchers; returns the normed output rows [T, hidden]."""
    L = LAYER
    ne, nh, nk, hd, nf, T = L["hidden"], L["heads"], L["kv_heads"], L["head_dim"], L["ffn"], L["tokens"]
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    h0 = c["h0"].to(dev)

    def norm(x, w):
        y = torch.empty_like(x)
        lib.launch_rms_norm_f32(x.data_ptr(), w.to(dev).data_ptr(), y.data_ptr(), ne, L["eps"], T, stream)
        torch.cuda.synchronize()
        return y

    def biased(x, w, b):
        y = host_product(x, w).to(dev).contiguous()
        lib.launch_add_bias_f32(y.data_ptr(), b.to(dev).data_ptr(), y.shape[1], T, stream)
        return y
    x = norm(h0, c["ln1"])
    q, k, v = biased(x, c["wq"], c["bq"]), biased(x, c["wk"], c["bk"]), biased(x, c["wv"], c["bv"])
    lib.launch_rope_f32(q.data_ptr(), nh, hd, T, L["theta"], 1.0, pos.data_ptr(), stream)
    lib.launch_rope_f32(k.data_ptr(), nk, hd, T, L["theta"], 1.0, pos.data_ptr(), stream)
    kc = torch.zeros(32, nk * hd, device=dev)
    vc = torch.zeros_like(kc)
    lib.launch_store_kv_f32(k.data_ptr(), kc.data_ptr(), nk * hd, T, pos.data_ptr(), stream)
    lib.launch_store_kv_f32(v.data_ptr(), vc.data_ptr(), nk * hd, T, pos.data_ptr(), stream)
    o = torch.empty(T, nh * hd, device=dev)
    lib.launch_gqa_attn_f32(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), pos.data_ptr(),
                            nh, nk, hd, 1.0 / hd ** 0.5, T, stream)
    torch.cuda.synchronize()
    a = host_product(o, c["wo"]).to(dev).contiguous()
    h1 = torch.empty_like(h0)
    lib.launch_add_f32(h0.data_ptr(), a.data_ptr(), h1.data_ptr(), h0.numel(), stream)
    x2 = norm(h1, c["ln2"])
    gate, up = host_product(x2, c["wg"]).to(dev).contiguous(), host_product(x2, c["wu"]).to(dev).contiguous()
    act = torch.empty_like(gate)
    lib.launch_swiglu_f32(gate.data_ptr(), up.data_ptr(), act.data_ptr(), gate.numel(), stream)
    torch.cuda.synchronize()
    d = host_product(act, c["wd"]).to(dev).contiguous()
    h2 = torch.empty_like(h0)
    lib.launch_add_f32(h1.data_ptr(), d.data_ptr(), h2.data_ptr(), h1.numel(), stream)
    return o.cpu().numpy(), h2.cpu().numpy(), norm(h2, c["final"]).cpu().numpy()


def main(lib_path: str, out_path: str) -> int:
    lib = ctypes.CDLL(lib_path)
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.launch_rms_norm_f32.argtypes = [vp, vp, vp, ci, cf, ci, vp]
    lib.launch_rope_f32.argtypes = [vp, ci, ci, ci, cf, cf, vp, vp]
    lib.launch_swiglu_f32.argtypes = [vp, vp, vp, ci, vp]
    lib.launch_store_kv_f32.argtypes = [vp, vp, ci, ci, vp, vp]
    lib.launch_gqa_attn_f32.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, cf, ci, vp]
    lib.launch_add_bias_f32.argtypes = [vp, vp, ci, ci, vp]
    lib.launch_add_f32.argtypes = [vp, vp, vp, ci, vp]
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
    out["layer_attention"], out["layer_residual"], out["layer_normed"] = run_layer(lib, c["layer"], dev, stream)
    np.savez_compressed(out_path, **out)
    print("wrote", out_path)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1], sys.argv[2]))
