"""Generate tests/golden/*.npz by running the reference's own torch fake-quant on CPU.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/nvfp4-training

It imports `small-model/model_ref.py` (pure torch, CPU) and stores seeded inputs together with the
outputs of `nvfp4_1d`, `nvfp4_2d`, `fp4_round`, `e4m3` and `hadamard16`.  The fixtures are what
pins `oracle/nvfp4_oracle.py`; nothing at test time needs the reference checkout.
"""
import os
import sys

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden.py /path/to/nvfp4-training")
ref_root = sys.argv[1]
sys.path.insert(0, os.path.join(ref_root, "small-model"))
import model_ref  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
torch.set_num_threads(1)


def bf16_bits(t):
    return t.bfloat16().view(torch.int16).numpy().view(np.uint16)


def student_t(g, shape, df=3):
    z = torch.randn(shape, generator=g)
    chi = torch.distributions.Chi2(torch.tensor(float(df)))
    torch.manual_seed(int(torch.randint(0, 2**31, (1,), generator=g)))
    v = chi.sample(shape)
    return z / torch.sqrt(v / df)


def inputs_1d():
    g = torch.Generator().manual_seed(0)
    cases = {}
    x = torch.randn(128, 256, generator=g)
    cols = torch.randperm(256, generator=g)[:4]
    x[:, cols] *= 30
    cases["normal_outliers"] = x
    cases["weights_small"] = torch.randn(128, 128, generator=g) * 0.02
    cases["student_t"] = student_t(g, (128, 192)) * 1e-3
    # many exact ties: small integers and halves
    cases["ties"] = torch.randint(-12, 13, (128, 64), generator=g).float() * 0.25
    # huge dynamic range: some blocks underflow to a zero scale byte, some to subnormal scales
    t = torch.randn(128, 128, generator=g)
    t[:, :32] *= 1e-6
    t[:, 32:64] *= 3e-4
    t[:, 64:80] = 0
    t[5, 100] = 1000.0
    cases["range"] = t
    cases["zeros"] = torch.zeros(128, 64)
    cases["tiny"] = torch.randn(128, 64, generator=g) * 1e-36
    cases["negzero"] = torch.where(torch.rand(128, 64, generator=g) < 0.3, -torch.zeros(128, 64), torch.randn(128, 64, generator=g))
    return {k: v.bfloat16() for k, v in cases.items()}


def main():
    out = {}
    # ---- scalar coders
    allbf = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).float()
    finite = torch.where(torch.isfinite(allbf), allbf, torch.zeros(()))
    out["fp4_round_all_bf16"] = model_ref.fp4_round(finite).numpy()
    pos16 = torch.arange(0x7C00, dtype=torch.int32).to(torch.int16).view(torch.float16).float()
    g = torch.Generator().manual_seed(1)
    rnd = torch.rand(20000, generator=g) * 500
    rnd2 = torch.rand(20000, generator=g) * 0.05
    ein = torch.cat([pos16, rnd, rnd2])
    out["e4m3_in"] = ein.numpy()
    out["e4m3_out"] = model_ref.e4m3(ein).numpy()
    out["hadamard16"] = model_ref.hadamard16("cpu").numpy()

    # ---- 1x16 row quantization
    for name, x in inputs_1d().items():
        out[f"rows_{name}_x"] = bf16_bits(x)
        out[f"rows_{name}_dq"] = model_ref.nvfp4_1d(x).numpy()
    # given amax (shared between two quantizations of the same tensor, llm-1b/model.py:60-66)
    x = inputs_1d()["student_t"]
    out["rows_gamax_dq"] = model_ref.nvfp4_1d(x, gamax=x.float().abs().max() * 4).numpy()

    # ---- 1x16 quantization with an exact PER-ROW scale (the contract of the operand emitters, llm-1b/emit.cu, and of
    # `q_rows` in small-model/qref.py:15-31, which is this formula row by row): each row is its own tensor
    xr = torch.cat([inputs_1d()["normal_outliers"][:24], inputs_1d()["student_t"][:24, :192].repeat(1, 2)[:, :256] * 1e3])
    xr[5] = 0
    out["rowscale_x"] = bf16_bits(xr)
    out["rowscale_dq"] = torch.cat([model_ref.nvfp4_1d(xr[r:r + 1]) for r in range(xr.shape[0])]).numpy()
    # the same with a GIVEN per-row scale (`q_rows_gs`, small-model/qref.py:33-42, without its column permutation),
    # through the reference's own `e4m3` / `fp4_round`: here twice the row's own scale, 1.0 for the all-zero row
    gs = xr.float().abs().amax(-1, keepdim=True) / 2688.0 * 2.0
    gs[5] = 1.0
    xb = (xr.float() / gs).reshape(xr.shape[0], xr.shape[1] // 16, 16)
    bs = model_ref.e4m3(xb.abs().amax(-1, keepdim=True) / 6.0)
    out["rowscale_gs"] = gs.reshape(-1).numpy()
    out["rowscale_gs_dq"] = ((model_ref.fp4_round(xb / bs.clamp(min=1e-30)) * bs).reshape(xr.shape) * gs).numpy()

    # ---- 16x16 weight quantization (bf16 weights as in llm-1b, fp32 as in small-model)
    g = torch.Generator().manual_seed(2)
    w = (torch.randn(128, 192, generator=g) * 0.02).bfloat16()
    out["w2d_bf16_w"] = bf16_bits(w)
    out["w2d_bf16_dq"] = model_ref.nvfp4_2d(w).numpy()
    out["w2d_bf16_dq_t"] = model_ref.nvfp4_2d(w.t().contiguous()).numpy()
    wf = torch.randn(256, 128, generator=g) / 128 ** 0.5
    wf[:16, :16] = 0
    out["w2d_f32_w"] = wf.numpy()
    out["w2d_f32_dq"] = model_ref.nvfp4_2d(wf).numpy()

    # ---- RHT16: integer-valued input so every summation order is exact in FP32
    g = torch.Generator().manual_seed(3)
    xi = torch.randint(-64, 65, (64, 128), generator=g).float().bfloat16()
    signs = 0b1010011010110001                       # llm-1b/model.py:42
    sv = torch.tensor([-1.0 if (signs >> i) & 1 else 1.0 for i in range(16)])
    H = model_ref.hadamard16("cpu") * sv[None, :]
    xt = xi.float().t()
    tr = (xt.reshape(xt.shape[0], -1, 16) @ H.t()).reshape(xt.shape)
    out["rht_int_x"] = bf16_bits(xi)
    out["rht_int_t"] = tr.numpy()
    out["rht_int_dq"] = model_ref.nvfp4_1d(tr, gamax=xi.float().abs().max() * 4).numpy()
    out["rht_signs"] = np.array([signs], dtype=np.uint32)
    # real-valued: matmul transform is only approximately the butterfly; stored for a tolerance check
    xr = (student_t(g, (64, 128)) * 1e-3).bfloat16()
    xt = xr.float().t()
    out["rht_real_x"] = bf16_bits(xr)
    out["rht_real_t"] = (xt.reshape(xt.shape[0], -1, 16) @ H.t()).reshape(xt.shape).numpy()

    np.savez_compressed(os.path.join(OUT, "model_ref_golden.npz"), **out)
    print("wrote", os.path.join(OUT, "model_ref_golden.npz"), {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
