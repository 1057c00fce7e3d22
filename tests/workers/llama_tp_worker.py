"""One rank of the tensor-parallel decoder test: the sharded model against the unsplit one it was made from (loss,
gradients of replicated parameters, gradients of each rank's slices)."""
import copy
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from dccl_b200 import Communicator  # noqa: E402
from dccl_b200.models.llama import LlamaConfig, LlamaDecoder  # noqa: E402
from dccl_b200.models.llama_tp import shard  # noqa: E402


def main():
    dev = "cpu"
    if "--cuda" in sys.argv[1:]:
        local = int(os.environ.get("DCCL_LOCAL_DEVICE", os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        comm = Communicator(device=local)
    else:
        comm = Communicator()
    n, r = comm.world, comm.rank
    torch.manual_seed(11)
    cfg = LlamaConfig(vocab_size=128, hidden=64, layers=2, heads=4, kv_heads=2 if n <= 2 else 4, ffn=96 if n != 4 else 128, max_seq=32)
    full = LlamaDecoder(cfg).to(dev)
    tokens = torch.randint(0, cfg.vocab_size, (2, 17)).to(dev)
    ref_loss = full.loss(tokens)
    ref_loss.backward()
    ok = True

    def check(a, b, what):
        nonlocal ok
        if not torch.allclose(a, b, rtol=2e-4, atol=2e-5):
            ok = False
            print("rank %d: %s differs by %g" % (r, what, (a - b).abs().max().item()))

    # plain form, and the form whose block exits write into pool buffers that are reduced in place
    for in_place, vocab in ((False, False), (True, False), (False, True), (True, True)):
        tag = ("in-place " if in_place else "") + ("vocab-parallel " if vocab else "")
        clean = copy.deepcopy(full)
        clean.zero_grad(set_to_none=True)
        tp = shard(clean, comm, in_place_reduce=in_place, vocab_parallel=vocab)
        loss = tp.loss(tokens)
        loss.backward()
        check(loss.detach(), ref_loss.detach(), tag + "loss")
        vs = slice(r * (cfg.vocab_size // n), (r + 1) * (cfg.vocab_size // n)) if vocab else slice(None)
        check(tp.embed.weight.grad, full.embed.weight.grad[vs], tag + "embedding gradient")
        check(tp.head.weight.grad, full.head.weight.grad[vs], tag + "head gradient")
        check(tp.norm.weight.grad, full.norm.weight.grad, tag + "final norm gradient")
        for i, (tb, fb) in enumerate(zip(tp.blocks, full.blocks)):
            check(tb.n1.weight.grad, fb.n1.weight.grad, tag + "block %d norm gradient" % i)
            qw = tb.attn.h * tb.attn.hd
            per = tb.gate.out_features
            check(tb.attn.q.weight.grad, fb.attn.q.weight.grad[r * qw:(r + 1) * qw], tag + "block %d q gradient" % i)
            check(tb.attn.o.weight.grad, fb.attn.o.weight.grad[:, r * qw:(r + 1) * qw], tag + "block %d o gradient" % i)
            check(tb.gate.weight.grad, fb.gate.weight.grad[r * per:(r + 1) * per], tag + "block %d gate gradient" % i)
            check(tb.down.weight.grad, fb.down.weight.grad[:, r * per:(r + 1) * per], tag + "block %d down gradient" % i)
        if dev != "cpu":
            torch.cuda.synchronize()
        tp.close()
    # sequence parallel: 16 positions split over the ranks; the ranks' loss shares add up to the loss, the replicated
    # parameters' gradients are partial sums until they are synchronised
    clean = copy.deepcopy(full)
    clean.zero_grad(set_to_none=True)
    sp = shard(clean, comm, sequence_parallel=True)
    part = sp.loss(tokens)
    part.backward()
    sp.sync_replicated_grads()
    whole = part.detach().clone()
    comm.all_reduce(whole, op="sum")
    check(whole, ref_loss.detach(), "sequence-parallel loss")
    check(sp.embed.weight.grad, full.embed.weight.grad, "sequence-parallel embedding gradient")
    check(sp.head.weight.grad, full.head.weight.grad, "sequence-parallel head gradient")
    check(sp.norm.weight.grad, full.norm.weight.grad, "sequence-parallel final norm gradient")
    for i, (tb, fb) in enumerate(zip(sp.blocks, full.blocks)):
        qw = tb.attn.h * tb.attn.hd
        per = tb.gate.out_features
        check(tb.n1.weight.grad, fb.n1.weight.grad, "sequence-parallel block %d norm gradient" % i)
        check(tb.n2.weight.grad, fb.n2.weight.grad, "sequence-parallel block %d second norm gradient" % i)
        check(tb.attn.q.weight.grad, fb.attn.q.weight.grad[r * qw:(r + 1) * qw], "sequence-parallel block %d q gradient" % i)
        check(tb.attn.o.weight.grad, fb.attn.o.weight.grad[:, r * qw:(r + 1) * qw], "sequence-parallel block %d o gradient" % i)
        check(tb.up.weight.grad, fb.up.weight.grad[r * per:(r + 1) * per], "sequence-parallel block %d up gradient" % i)
        check(tb.down.weight.grad, fb.down.weight.grad[:, r * per:(r + 1) * per], "sequence-parallel block %d down gradient" % i)

    if dev != "cpu":
        torch.cuda.synchronize()
    comm.finalize()
    if not ok:
        sys.exit(1)
    print("OK llama tp worker rank %d" % r)


if __name__ == "__main__":
    main()
