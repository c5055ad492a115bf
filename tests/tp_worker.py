"""One rank of the tensor-parallel GPU test (tests/test_gpu_tp.py starts one process per GPU):
python -m tests.tp_worker <rank> <world> <id file> <out file> <steps>."""
import os
import sys
import time

import numpy as np

from vexel_b200 import capi, gguf_synth as gs, tp

SPEC = gs.scaled(gs.C2_LLAMA2_7B, 2, 512, 8, 4, 64, 1024, 2048)
SEED = 21
PROMPTS = {1: 37, 2: 5, 3: 64}


def prompt(seq, n):
    return np.random.default_rng(100 + seq).integers(0, SPEC.vocab, n).astype(np.int32)


def main():
    rank, world, id_file, out_file, steps = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], int(sys.argv[5])
    be = capi.Backend(rank)
    be.lib.vx_set_graphs(int(os.environ.get("VEXEL_TP_GRAPHS", "0")))
    if rank == 0:                                   # the id comes from the NCCL build the ranks themselves run
        with open(id_file + ".tmp", "wb") as f:
            f.write(tp.unique_id(be))
        os.replace(id_file + ".tmp", id_file)
    deadline = time.time() + 120
    while not os.path.exists(id_file):
        if time.time() > deadline:
            raise TimeoutError("rank 0 never published the NCCL id")
        time.sleep(0.05)
    tp.init(be, open(id_file, "rb").read(), rank, world)
    m = tp.load_sharded(be, SPEC, gs.synth_tensors(SPEC, SEED), rank, world,
                        max_blocks=64, max_seqs=8, max_batch_tokens=128, max_blocks_per_seq=16)
    toks = {}
    last = {}
    for s, n in PROMPTS.items():
        m.seq_create(s)
        last[s] = int(m.prefill(s, prompt(s, n)))
        toks[s] = [last[s]]
    pos = dict(PROMPTS)
    ids = np.array(sorted(PROMPTS), np.int64)
    first_logits = None
    for _ in range(steps):
        out, logits = m.decode_step(ids, np.array([last[int(s)] for s in ids], np.int32), [pos[int(s)] for s in ids], want_logits=True)
        if first_logits is None:
            first_logits = np.array(logits)
        for s, t in zip(ids, out):
            last[int(s)] = int(t); toks[int(s)].append(int(t)); pos[int(s)] += 1
    np.savez(out_file, tokens=np.array([toks[int(s)] for s in ids]), logits=first_logits)
    m.close(); tp.shutdown(be); be.close()


if __name__ == "__main__":
    main()
