"""Child process of tests/test_gpu_tp.py: one tensor-parallel rank on its own GPU (NCCL, NVLS off)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "let-it-slide_b200"))


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    import datetime
    # a short collective timeout: if the peer rank dies, this rank's next collective errors out instead of waiting
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))
    from rptc_b200 import ops
    from rptc_b200.llama import LlamaConfig, RPTCLlama
    chain = sys.argv[5] if len(sys.argv) > 5 else "fused"
    if chain == "glued":        # norms inside the matvecs: needs 4096-wide rows
        cfg = LlamaConfig(hidden=4096, layers=2, heads=32, kv_heads=8, ffn=2048, vocab=512, max_pos=16, weight_scale=0.02)
    else:
        cfg = LlamaConfig(hidden=1024, layers=2, heads=8, kv_heads=2, ffn=2048, vocab=512, max_pos=16, weight_scale=0.05)
    rows, T = 2, 6
    use_peer = len(sys.argv) > 4 and sys.argv[4] == "peer"
    model = RPTCLlama(cfg, rows=rows, seed=3, tp_world=world, tp_rank=rank, peer_allreduce=use_peer)
    model.fused_tp = chain != "unfused"
    model.glued_tp = chain == "glued"            # (hidden 1024 cannot take it anyway)
    assert model._fusable_tp() == model.fused_tp
    g = torch.Generator(device="cuda").manual_seed(5)                    # same tokens on every rank
    tokens = torch.randint(0, cfg.vocab, (rows, T), device="cuda", generator=g)
    ref = model.reference_logits(tokens)
    print(f"rank {rank}: reference done", flush=True)
    worst = 0.0
    for use_graph in (False, True):
        model.reset()
        if use_graph:
            model.capture(pdl=True)
        print(f"rank {rank}: graph={use_graph} ready", flush=True)
        for t in range(T):
            model.ids.copy_(tokens[:, t].to(torch.int32))
            model.step()
            torch.cuda.synchronize()
            err = (model.logits.float() - ref[:, t]).abs().max().item() / ref[:, t].abs().max().item()
            worst = max(worst, err)
    ops.device_status()
    same = torch.tensor([model.logits.float().sum().item()], device="cuda", dtype=torch.float64)
    lo, hi = same.clone(), same.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    # graphs that captured collectives must be gone before their communicator is torn down
    model.graph = None
    torch.cuda.synchronize()
    if model.peer is not None:
        model.peer.close()
    print(f"rank {rank}: worst {worst:.2e}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    assert worst <= (2e-2 if chain == "glued" else 1e-2), f"rank {rank}: logits off by {worst}"
    assert abs(hi.item() - lo.item()) <= 1e-3 * abs(hi.item()) + 1e-3, "ranks disagree on the logits"
    print(f"rank {rank} ok worst {worst:.2e}")


if __name__ == "__main__":
    main()
