"""Worker of tests/test_gpu_tp.py: one rank of a 2-GPU tensor-parallel toy decoder.  Decodes a few tokens
with NCCL all-reduces and again with the all-reduce fused into the norm kernel, and checks that both
agree and that no bounded wait ran out.  Launched with RANK / WORLD_SIZE / MASTER_* in the environment."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    config_name = os.environ.get("TX_TP_CONFIG", "toy128")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from texelator_b200.modeling import CONFIGS, BC4Decoder
    model = BC4Decoder(CONFIGS[config_name], f"cuda:{rank}", max_len=400, seed=5, tp_rank=rank, tp_world=world)
    ids = torch.randint(0, model.config.vocab, (200,), generator=torch.Generator().manual_seed(2))
    model.prefill(ids)
    model.tok.fill_(int(ids[-1]))
    state = (model.tok.clone(), model.pos.clone(), model.mask.clone(), model.k_cache.clone(), model.v_cache.clone())

    def run(steps, single=False):
        model.tok.copy_(state[0]); model.pos.copy_(state[1]); model.mask.copy_(state[2])
        model.k_cache.copy_(state[3]); model.v_cache.copy_(state[4])
        hidden, tokens = [], []
        for _ in range(steps):
            model.decode_eager(fused=not single, single=single)
            hidden.append(model.last_hidden.float().clone()); tokens.append(int(model.next_tok))
        return hidden, tokens

    ref_hidden, ref_tokens = run(4)
    ok = model.enable_peer_exchange()
    if not ok:
        print(f"rank {rank}: peer exchange unavailable", flush=True)
        dist.barrier()
        os._exit(3)
    model.ext.kernel_status(clear=True)
    hidden, tokens = run(4)
    # second generation: packets pushed from the linears' epilogues, cluster reduce, token packets
    assert model.single
    hidden2, tokens2 = run(4, single=True)
    worst2 = min(float(torch.nn.functional.cosine_similarity(a.reshape(1, -1), b.reshape(1, -1))) for a, b in zip(hidden2, ref_hidden))
    worst = min(float(torch.nn.functional.cosine_similarity(a.reshape(1, -1), b.reshape(1, -1))) for a, b in zip(hidden, ref_hidden))
    # graph replay of the same path
    model.tok.copy_(state[0]); model.pos.copy_(state[1]); model.mask.copy_(state[2])
    model.k_cache.copy_(state[3]); model.v_cache.copy_(state[4])
    model.capture()
    graph_tokens = []
    for _ in range(4):
        model.decode_graph()
        torch.cuda.synchronize()
        graph_tokens.append(int(model.next_tok))
    status = model.ext.kernel_status()
    # every rank must hold the same bits (rank-ordered sum)
    mine = model.last_hidden.float().clone()
    other = mine.clone()
    dist.broadcast(other, src=0)
    same_bits = bool(torch.equal(mine, other))
    print(f"rank {rank}: cosine {worst:.6f} / {worst2:.6f} tokens {tokens} / {tokens2} ref {ref_tokens} graph {graph_tokens} status {status} "
          f"same_bits {same_bits}", flush=True)
    good = (worst >= 0.9995 and worst2 >= 0.9995 and tokens == ref_tokens and tokens2 == ref_tokens and graph_tokens == tokens
            and status == 0 and same_bits)
    model.graph = None
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0 if good else 1)


if __name__ == "__main__":
    main()
