"""Generate the golden fixtures in this directory from the reference project itself.

Run once, in a container where the reference checkout is importable:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own `qfactory.convert.convert_params` (the packer) and the
`asymmetric_quant` / `dequant` helpers of its `tests/acc_gptq.py` (importable because
that file's body is guarded by `__main__`), feeds them small seeded inputs and stores
inputs and outputs as .npz files of a few KB each.  The fixtures travel with the
repository; the reference checkout does not have to exist where the tests run.

Cases
  pack_b{2,4,8}_*      convert_params on codes/scales/zeros (asym, sym, group-less)
  dequant_b{2,4,8}     dequant() + fp16 matmul on randn activations
  quant_b{2,4,8}       asymmetric_quant() of a randn fp16 weight, then dequant()
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    sys.path.insert(0, root)
    from qfactory.convert import convert_params  # noqa: E402

    spec = importlib.util.spec_from_file_location("ref_acc_gptq", os.path.join(root, "tests", "acc_gptq.py"))
    acc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(acc)
    return convert_params, acc.asymmetric_quant, acc.dequant


def main(root):
    convert_params, asymmetric_quant, dequant = load_reference(root)
    for bits in (2, 4, 8):
        g = torch.Generator().manual_seed(100 + bits)
        K, N, GS = 512, 48, 64
        q = torch.randint(0, 1 << bits, (K, N), generator=g, dtype=torch.int32)
        s = (torch.rand(K // GS, N, generator=g) * 0.018 + 0.002).to(torch.float16)
        z = torch.randint(0, 1 << bits, (K // GS, N), generator=g, dtype=torch.int32)
        # make sure both ends of the zero range (the clamp at 2^b-1 and zero) are hit
        z[0, 0], z[0, 1] = (1 << bits) - 1, 0
        q[0, 0], q[1, 0] = 0, (1 << bits) - 1
        w_a, s_a, z_a = convert_params({"K": K, "N": N, "NBITS": bits, "GS": GS}, (q, s, z))
        w_s, s_s, z_s = convert_params({"K": K, "N": N, "NBITS": bits, "GS": GS}, (q, s, None))
        assert z_s is None
        w_g = convert_params({"K": K, "N": N, "NBITS": bits}, (q,))
        np.savez_compressed(
            os.path.join(HERE, f"pack_b{bits}.npz"),
            K=K, N=N, GS=GS, bits=bits,
            q=q.numpy(), s=s.numpy(), z=z.numpy(),
            w_asym=w_a.numpy(), s_asym=s_a.numpy(), z_asym=z_a.numpy(),
            w_sym=w_s.numpy(), s_sym=s_s.numpy(), w_groupless=w_g.numpy(),
        )

        # dequant + fp16 matmul, zeros kept below 2^b-1 so the clamp is not in play
        M = 3
        x = torch.randn(M, K, generator=g).to(torch.float16)
        z2 = torch.randint(0, (1 << bits) - 1, (K // GS, N), generator=g, dtype=torch.int32)
        wd = dequant(q, s, z2)
        y = x @ wd
        yg = x @ q.to(torch.float16)
        np.savez_compressed(
            os.path.join(HERE, f"dequant_b{bits}.npz"),
            K=K, N=N, GS=GS, bits=bits, M=M,
            x=x.numpy(), q=q.numpy(), s=s.numpy(), z=z2.numpy(),
            wdq=wd.numpy(), y=y.numpy(), y_groupless=yg.numpy(),
        )

        # fp16 -> codes front end
        wf = torch.randn(256, 24, generator=g).to(torch.float16)
        qq, ss, zz = asymmetric_quant(wf, 64, bits)
        wd2 = dequant(qq, ss, zz)
        np.savez_compressed(
            os.path.join(HERE, f"quant_b{bits}.npz"),
            bits=bits, GS=64, w=wf.numpy(), q=qq.numpy(), s=ss.numpy(), z=zz.numpy(), wdq=wd2.numpy(),
        )
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("QF_REFERENCE_ROOT", ""))
