"""Worker of tests/test_gpu_tp_parity.py: a few training steps of a d=1024 hybrid model at TP = WORLD_SIZE on the same
seeded batch, with the fused compute + collective kernels on; every rank writes its losses, a digest of every replicated
parameter and the device status word to ``<out>.<rank>.pt``."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out, steps = sys.argv[1], int(sys.argv[2])
    fused = sys.argv[3] == "1" if len(sys.argv) > 3 else True
    from hippolm_b200.cli import build_parser
    from hippolm_b200.train.loop import setup_worker, train_step, teardown_worker
    from hippolm_b200.data.packing import synthetic_packed_batch
    from hippolm_b200.ops import _ext
    a = build_parser().parse_args([])
    a.vocab_size, a.hidden_size, a.num_heads, a.head_dim = 8192, 1024, 8, 128
    a.num_layers, a.num_blocks, a.intermediate_size = 4, 2, 2048
    a.ffn_nvfp4 = a.ffn_nvfp4_no_bf16_master = False
    a.batch_size, a.seq_len, a.micro_batch_size, a.max_steps = 4, 1024, 2048, 1000
    a.tp_size, a.dp_size, a.fused_comm, a.seed = int(os.environ.get("WORLD_SIZE", "1")), 1, fused, 7
    a.muon_ns_scope = "full"
    a.dist_timeout_s = 120
    ctx = setup_worker(a, run_dir=None, data_iter=iter(()))
    ids, labels, cu = synthetic_packed_batch(4 * 1024, 8192, 5, 128, 1024, row_len=1024)
    batch = {"input_ids": ids, "labels": labels, "cu_seqlens": cu, "row_len": 1024}
    losses = []
    for _ in range(steps):
        losses.append(float(train_step(ctx, batch)["loss"])); ctx.step += 1
    torch.cuda.synchronize()
    rep = {n: p.detach().float().cpu() for n, p in ctx.model.named_parameters() if getattr(p, "tp_replicated", False)}
    torch.save({"losses": losses, "replicated": rep, "status": tuple(_ext.device_status()),
                "fused": bool(ctx.extras.get("fused_comm", False))}, f"{out}.{ctx.mesh.rank}.pt")
    teardown_worker(ctx)


if __name__ == "__main__":
    main()
