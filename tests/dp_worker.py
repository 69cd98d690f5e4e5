"""Worker of the multi-GPU tests: trains a small hybrid model for a few steps under torchrun and writes rank 0's final
parameters and loss trace to the path in argv[1]. argv[2]: 'fused' or 'nccl' (the data-parallel step implementation)."""

import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
os.environ["GHB_COMM"] = sys.argv[2]

import torch  # noqa: E402

from gdn_hybrid_architecture_ideas_b200 import config as C  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.ops import native  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.parallel import data_parallel  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer  # noqa: E402


def main():
    dp = data_parallel.from_environment()
    model = C.hybrid_model_config("60m", full=True)
    model.encoder.n_layers, model.encoder.nope_global_layers, model.vocab_size = 4, (0,), 4096
    cfg = C.TrainConfig(model=model, data=C.DataConfig(kind="uniform", seq_len=256, batch_size=2 * dp.world, seed=5), steps=100, seed=7)
    cfg.autocast, cfg.head_impl, cfg.metrics_jsonl, cfg.log_every, cfg.optimizer_sharding = "bfloat16", "fused", False, 0, "zero2"
    cfg.optim.warmup_steps, cfg.optim.lr = 1, 1e-4     # small steps: Adam's sign-like first updates would amplify rounding noise
    t = Trainer(cfg, None, dp)
    losses = [t.train_step()["loss"] for _ in range(3)]
    native.check_status()
    fused = t.zero is not None and t.zero.fused is not None
    lp_before = t.flat.lp.detach().float().cpu().clone()      # the bf16 compute weights are complete on every rank after a step
    t.zero.gather_master()                                    # fp32 masters of the matrices live on their owners until gathered
    torch.cuda.synchronize()
    by_name = {n: t.flat.view(t.flat.params, n).detach().cpu().clone() for n in t.flat.by_name}       # by name: the two runs may lay the buffer out differently
    lp_by_name = {n: lp_before[t.flat.by_name[n].offset:t.flat.by_name[n].offset + t.flat.by_name[n].numel].clone() for n in t.flat.by_name}
    if dp.lead:
        torch.save({"losses": losses, "fused": fused, "multimem": bool(fused and t.zero.fused.multimem), "early": t.zero.early,
                    "params": by_name, "lp": lp_by_name}, sys.argv[1])
    dp.barrier()
    dp.close()


if __name__ == "__main__":
    main()
