"""Worker of test_two_gpu_sharded_run_matches_single_gpu (launched with torchrun, 2 ranks)."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(out_dir):
    from onecompression_b200 import GPTQ, QEPConfig, synthetic
    from onecompression_b200.qep._quantize_with_qep_arch import BlockQuantizer
    from onecompression_b200.sharding import ShardedContext, seq_shard

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    shape = dict(synthetic.LLAMA3_8B, hidden_size=256, intermediate_size=512, num_attention_heads=4,
                 num_key_value_heads=2, head_dim=64, vocab_size=1000)

    def run(ctx, rows):
        stack = synthetic.llama_blocks(shape, 1, 64, dev, seed=11)
        x0 = synthetic.embedded_tokens(1000, 256, 48, 64, dev, seed=11, row_range=rows) * 30
        q = GPTQ(wbits=4, groupsize=128, sym=False)
        for n, m in stack.blocks[0].named_modules():
            if isinstance(m, torch.nn.Linear):
                q.module_to_name[m] = f"model.layers.0.{n}"
        runner = BlockQuantizer(q, QEPConfig(device=str(dev)), batch_size=16, device=dev, dist=ctx)
        nq, _ = runner.run(stack.blocks[0], x0.clone(), x0.clone(), stack.kwargs)
        return q.results, nq

    sharded, nq_s = run(ShardedContext(), seq_shard(48, rank, world))
    single, nq_1 = run(None, None)
    total = match = 0
    for name, r in single.items():
        s = sharded[name]
        a = torch.from_numpy(__import__("numpy").asarray(r.qweight))
        total += a.numel()
        match += int((a == s.qweight).sum())
        assert s.qweight.shape == r.qweight.shape and s.qzeros.shape == r.qzeros.shape
        assert s.scales.shape == r.scales.shape
    frac = match / total
    # packed words: a word differs if any of its 8 codes differs
    assert frac >= 0.99, frac
    a, b = seq_shard(48, rank, world)
    rel = ((nq_s.float() - nq_1[a:b].float()).norm() / nq_1[a:b].float().norm()).item()
    assert rel < 0.05, rel
    dist.barrier()
    if rank == 0:
        open(os.path.join(out_dir, "ok"), "w").write(f"{frac} {rel}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
