"""Worker of the tensor-parallel model tests (one process per rank under torchrun): a tensor-parallel Trainer step on
weights cut from a full model equals the full model's loss and gradients computed in the same process.
argv[1]: output path."""

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402

from gdn_hybrid_architecture_ideas_b200 import config as C  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.models import build_model  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.parallel import data_parallel, tp_model  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.train.fused_head import chunked_ce  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer  # noqa: E402


def main():
    dp = data_parallel.from_environment()
    dev = dp.device
    cuda = dev.type == "cuda"
    model = C.hybrid_model_config("60m", full=True)
    model.encoder.n_layers, model.encoder.nope_global_layers, model.vocab_size = 4, (0,), 1024
    if cuda:
        model.d_model, model.ffn_hidden = 256, 512
        model.encoder.gdn.n_k_heads = model.encoder.gdn.n_v_heads = dp.world
        model.encoder.attention.n_q_heads, model.encoder.attention.n_kv_heads = 2 * dp.world, dp.world
        seq, rows = 256, dp.world
    else:
        model.d_model, model.ffn_hidden = 64, 32 * dp.world
        g = model.encoder.gdn
        g.n_k_heads = g.n_v_heads = dp.world
        g.k_head_dim, g.v_head_dim = 16, 32
        a = model.encoder.attention
        a.n_q_heads, a.n_kv_heads, a.head_dim = 2 * dp.world, dp.world, 16
        seq, rows = 32, 2
    cfg = C.TrainConfig(model=model, data=C.DataConfig(kind="uniform", seq_len=seq, batch_size=rows, seed=5), steps=10, seed=3)
    cfg.metrics_jsonl, cfg.log_every, cfg.head_impl = False, 0, "fused" if cuda else "chunked"
    cfg.autocast = "bfloat16" if cuda else "none"
    cfg.tensor_parallel = dp.world

    torch.manual_seed(3)
    full = build_model(cfg.model).to(dev)
    t = Trainer(cfg, None, dp)
    t.model.load_state_dict(tp_model.shard_state_dict(full.state_dict(), cfg.model, dp.rank, dp.world))
    t.flat.refresh_lp()
    batch = t.batch_at(0).to(dev)
    n = int(batch.target_valid.sum())

    # the full model on the whole batch, in this process
    if cuda:
        from gdn_hybrid_architecture_ideas_b200 import ops
        ops.set_mode("reference")
    with torch.autocast(dev.type, dtype=torch.bfloat16, enabled=cuda):
        hidden = full(batch.tokens, batch.doc_ids, return_hidden=True).hidden_aux
    valid = batch.target_valid.float()
    loss_full, _ = chunked_ce(hidden, full.head_weight(), batch.targets, valid / n, valid * (cfg.loss.z_loss / n))
    loss_full.backward()
    if cuda:
        ops.set_mode("native")
    gnorm_full = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in full.parameters() if p.grad is not None))
    want = tp_model.shard_state_dict({k: p.grad for k, p in full.named_parameters()}, cfg.model, dp.rank, dp.world)

    out = t.device_step(batch, n, lr=0.0)
    got = {k: p.grad.detach().float().cpu().clone() for k, p in t.model.named_parameters()}
    if cuda:
        from gdn_hybrid_architecture_ideas_b200.ops import native
        torch.cuda.synchronize()
        native.check_status()
    torch.save({"loss": float(out[0]), "gnorm": float(out[2]), "loss_full": float(loss_full), "gnorm_full": float(gnorm_full),
                "got": got, "want": {k: v.detach().float().cpu() for k, v in want.items()}}, f"{sys.argv[1]}.{dp.rank}")
    dp.barrier()
    dp.close()


if __name__ == "__main__":
    main()
