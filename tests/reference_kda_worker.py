"""Child process of ``test_reference_kda_op.py``: the reference's token-recurrent KDA kernel
(``fla/ops/kda/fused_recurrent.py``, run by Triton's interpreter on the CPU) on packed documents with initial states,
in-kernel L2 normalisation and in-kernel gate activation; inputs and outputs go to a file."""
import contextlib
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
import torch  # noqa: E402

torch.cpu.device = lambda index=None: contextlib.nullcontext()


def inputs(case: int):
    g = torch.Generator().manual_seed(100 + case)
    H, K = (2, 32) if case % 2 == 0 else (3, 64)
    lens = [[37, 5, 64, 22], [130], [1, 1, 90]][case % 3]
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()))
    r = lambda *s: torch.randn(*s, generator=g)                       # noqa: E731
    d = dict(q=r(1, T, H, K), k=r(1, T, H, K), v=r(1, T, H, K), x_g=r(1, T, H, K), beta=torch.sigmoid(r(1, T, H)),
             A_log=0.3 * r(H), dt_bias=0.5 * r(H * K), h0=0.2 * r(len(lens), H, K, K), cu=cu,
             lower_bound=[None, -5.0, -1.5][case % 3])
    return d


def main():
    ref_root, out = sys.argv[1], sys.argv[2]
    sys.path.insert(0, ref_root)
    from src.models.ops._vendored.fla.ops.kda.fused_recurrent import fused_recurrent_kda
    res = []
    for case in range(6):
        d = inputs(case)
        o, ht = fused_recurrent_kda(q=d["q"], k=d["k"], v=d["v"], g=d["x_g"], beta=d["beta"], A_log=d["A_log"],
                                    dt_bias=d["dt_bias"], initial_state=d["h0"].clone(), output_final_state=True,
                                    use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, lower_bound=d["lower_bound"],
                                    cu_seqlens=d["cu"])
        res.append((o.float(), ht.float()))
    torch.save(res, out)


if __name__ == "__main__":
    main()
