"""Tensor-parallel decode on two GPUs against the CPU oracle running the whole model.

One process per GPU (tests/tp_worker.py), each holding half of every projection, half of the KV heads and half of the
output head; the partial Wo / W2 outputs meet in NCCL all-reduces, the two local maxima in one all-gather.  Both ranks must
emit the same greedy tokens, those tokens must be the oracle's, and the two logits slices side by side must be the
oracle's logits within the step tolerance.  NVLS is switched off for the run: no memory of these short-lived processes is
bound to a multicast object."""
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import oracle_config, rel_l2
from tests import tp_worker as W
from vexel_b200 import capi, gguf_synth as gs, tp

pytestmark = pytest.mark.gpu
STEPS = 24


def _gpu_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("graphs", [0, 1], ids=["eager", "graph-replay"])
def test_two_rank_greedy_decode_matches_oracle(be, tmp_path, graphs):
    world = 2
    id_file = tmp_path / "nccl_id.bin"                                             # written by rank 0
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", VEXEL_TP_GRAPHS=str(graphs))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = [subprocess.Popen([sys.executable, "-m", "tests.tp_worker", str(r), str(world), str(id_file),
                               str(tmp_path / f"rank{r}.npz"), str(STEPS)], cwd=root, env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=300)[0])
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"rank {r} failed:\n{outs[r][-3000:]}"
    res = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    assert np.array_equal(res[0]["tokens"], res[1]["tokens"])                     # one global argmax, seen by both ranks

    spec = W.SPEC
    om = O.Model(oracle_config(spec, 64))
    for layer, slot, t, raw in gs.synth_tensors(spec, W.SEED):
        if layer < 0: om.set_global(slot, t, raw)
        else: om.set_layer(layer, slot, t, raw)
    ids = sorted(W.PROMPTS)
    want = []
    first = []
    for s in ids:
        om.pool.create_seq(s)
        n = W.PROMPTS[s]
        lg = om.forward(s, W.prompt(s, n), 0)
        seq = [O.argmax(lg[-1] if lg.ndim == 2 else lg)]
        for i in range(STEPS):
            lg = om.forward(s, np.array([seq[-1]], np.int32), n + i)
            lg = lg[-1] if lg.ndim == 2 else lg
            if i == 0:
                first.append(np.array(lg))
            seq.append(O.argmax(lg))
        want.append(seq)
    want = np.array(want)
    got = res[0]["tokens"]
    agree = float((got == want).mean())
    logits = np.concatenate([res[0]["logits"], res[1]["logits"]], axis=1)         # vocabulary halves side by side
    err = max(rel_l2(logits[i], first[i]) for i in range(len(ids)))
    print(f"TP-2: greedy agreement {agree:.3f} over {want.size} tokens, first-step logits rel-L2 {err:.2e}")
    assert err < 1e-3
    assert np.array_equal(got[:, :2], want[:, :2])                                # prefill and the first step exactly
    assert agree >= 0.95
