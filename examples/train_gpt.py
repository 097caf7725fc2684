"""Train a GPT with any mesh / quantisation / offload setting.

    python examples/train_gpt.py --steps 200
    torchrun --nproc_per_node=8 examples/train_gpt.py --dp-shard 8 --ac selective --dim 1024 --layers 24
    torchrun --nproc_per_node=8 examples/train_gpt.py --dp-replicate 8 --ep 8 --experts 8
"""
import argparse

import forgeminds_b200 as fm


def main():
    p = argparse.ArgumentParser()
    for name, default in (("steps", 200), ("dim", 256), ("layers", 4), ("heads", 8), ("kv-heads", 4), ("seq", 256),
                          ("micro-batch", 8), ("grad-accum", 1), ("dp-replicate", 1), ("dp-shard", 1), ("tp", 1),
                          ("pp", 1), ("ep", 1), ("experts", 0)):
        p.add_argument(f"--{name}", type=int, default=default)
    p.add_argument("--quant", default="none", choices=["none", "fp8", "int8", "int8_wo"])
    p.add_argument("--ac", default="none", choices=["none", "full", "selective"])
    p.add_argument("--optimizer", default="adamw", choices=["adamw", "muon"])
    p.add_argument("--offload-opt", action="store_true")
    p.add_argument("--offload-act", action="store_true")
    p.add_argument("--ckpt-dir", default="checkpoints")
    p.add_argument("--ckpt-every", type=int, default=0)
    a = p.parse_args()

    cfg = fm.ForgeConfig()
    cfg.parallel.__dict__.update(dp_replicate=a.dp_replicate, dp_shard=a.dp_shard, tp=a.tp, pp=a.pp, ep=a.ep)
    cfg.quant.mode = a.quant
    cfg.offload.optimizer, cfg.offload.activations = a.offload_opt, a.offload_act
    cfg.train.__dict__.update(max_steps=a.steps, grad_accum=a.grad_accum, ac=a.ac, optimizer=a.optimizer,
                              ckpt_dir=a.ckpt_dir, ckpt_every=a.ckpt_every)
    mc = fm.GPTConfig(vocab_size=32000, dim=a.dim, n_layers=a.layers, n_heads=a.heads, n_kv_heads=a.kv_heads,
                      max_seq=a.seq, n_experts=a.experts)
    data = fm.SyntheticLM(mc.vocab_size, a.seq, n=8192)
    trainer = fm.Trainer(lambda ctx: fm.GPT(mc, fm.moe_kwargs(ctx, cfg) if a.experts else None), cfg, data,
                         micro_batch=a.micro_batch)
    trainer.fit()
    trainer.close()
    fm.cleanup()


if __name__ == "__main__":
    main()
