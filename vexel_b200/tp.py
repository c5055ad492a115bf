"""Tensor parallelism over NCCL for models that one GPU cannot hold (or serve fast enough): host-side sharding helpers.

The reference keeps every projection of a block whole on one device (inference/runtime/block.go:256-266) and has no
multi-GPU path, so this module mirrors no reference interface; it prepares what the library's tensor-parallel step expects
(include/vexel_cuda.h, "tensor parallelism"):

  * Wq / Wk / Wv, W1 / W3 and the output head are split by OUTPUT rows (whole attention heads, FFN columns, vocabulary
    rows): rank r keeps rows [r*N/W, (r+1)*N/W) of the GGUF tensor -- whole byte rows, no re-quantisation;
  * Wo and W2 are split by INPUT columns, on GGUF block boundaries (32 weights for Q4_0, 256 for the K-quants): rank r keeps
    blocks [r*Kb/W, (r+1)*Kb/W) of every row; the partial outputs are summed over the ranks by one all-reduce each;
  * the embedding table and the norm vectors are replicated.

Every rank then runs the same greedy step on the same token ids; a rank's KV pool holds its own KV heads only.
"""
import ctypes as C
import dataclasses

import numpy as np

from . import capi

# GGUF block geometry: type -> (weights per block, bytes per block)   (inference/pkg/gguf/dequant.go:14-31)
BLOCK = {capi.T_F32: (1, 4), capi.T_Q4_0: (32, 18), capi.T_Q4_K: (256, 144), capi.T_Q6_K: (256, 210)}

ROW_SPLIT = (capi.W_WQ, capi.W_WK, capi.W_WV, capi.W_W1, capi.W_W3)     # by output rows
COL_SPLIT = (capi.W_WO, capi.W_W2)                                      # by input columns (GGUF blocks)
UNIQUE_ID_BYTES = 128


def check_divisible(spec, world):
    """Raises ValueError unless every split lands on a head / GGUF-block boundary."""
    from . import gguf_synth as gs
    proj_types, _, out_type = gs.tensor_types(spec)
    if spec.n_heads % world or spec.n_kv_heads % world:
        raise ValueError(f"{spec.n_heads} query / {spec.n_kv_heads} KV heads do not divide over {world} ranks")
    if spec.ffn % world or spec.vocab % world:
        raise ValueError(f"FFN width {spec.ffn} or vocabulary {spec.vocab} does not divide over {world} ranks")
    for slot, k in ((capi.W_WO, spec.n_heads * spec.head_dim), (capi.W_W2, spec.ffn)):
        per = BLOCK[proj_types[slot]][0]
        if (k // world) % per:
            raise ValueError(f"slot {slot}: {k} input columns over {world} ranks is not a whole number of {per}-weight blocks")


def local_spec(spec, world):
    """The shape one rank's model is created with: local head, FFN and vocabulary counts."""
    check_divisible(spec, world)
    return dataclasses.replace(spec, n_heads=spec.n_heads // world, n_kv_heads=spec.n_kv_heads // world,
                               ffn=spec.ffn // world, vocab=spec.vocab // world)


def shard_rows(raw, rank, world):
    """Rows [rank*N/W, (rank+1)*N/W) of a [N, bytes-per-row] GGUF tensor."""
    n = raw.shape[0]
    assert n % world == 0
    return np.ascontiguousarray(raw[rank * n // world:(rank + 1) * n // world])


def shard_cols(raw, type_id, rank, world):
    """GGUF blocks [rank*Kb/W, (rank+1)*Kb/W) of every row of a [N, Kb * block bytes] tensor."""
    _, nbytes = BLOCK[type_id]
    n = raw.shape[0]
    r = raw.reshape(n, -1)
    if type_id == capi.T_F32:
        r = r.view(np.uint8).reshape(n, -1)
    kb = r.shape[1] // nbytes
    assert r.shape[1] == kb * nbytes and kb % world == 0
    out = np.ascontiguousarray(r.reshape(n, kb, nbytes)[:, rank * kb // world:(rank + 1) * kb // world]).reshape(n, -1)
    return out.view(np.float32) if type_id == capi.T_F32 else out


def shard_tensor(layer, slot, type_id, raw, rank, world):
    """This rank's slice of one model tensor (layer -1 = globals)."""
    if layer < 0:
        return shard_rows(raw, rank, world) if slot == capi.G_OUTPUT else raw
    if slot in ROW_SPLIT:
        return shard_rows(raw, rank, world)
    if slot in COL_SPLIT:
        return shard_cols(raw, type_id, rank, world)
    return raw                                                          # norm vectors


def unique_id(be):
    """The NCCL id rank 0 creates and hands to the other ranks (any channel: a file, a store, a broadcast)."""
    buf = (C.c_ubyte * UNIQUE_ID_BYTES)()
    be._ck(be.lib.vx_tp_unique_id(buf, UNIQUE_ID_BYTES))
    return bytes(buf)


def init(be, uid, rank, world):
    buf = (C.c_ubyte * UNIQUE_ID_BYTES).from_buffer_copy(uid)
    be._ck(be.lib.vx_tp_init(be.h, buf, rank, world))


def init_from_torch(be, dist):
    """Joins the ranks of an initialised torch.distributed group (any backend) into one NCCL communicator of the library's own."""
    rank, world = dist.get_rank(), dist.get_world_size()
    box = [unique_id(be) if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    init(be, box[0], rank, world)
    return rank, world


def shutdown(be):
    be._ck(be.lib.vx_tp_shutdown(be.h))


def create_model(be, spec, world, max_blocks, max_seqs, max_batch_tokens, max_blocks_per_seq):
    """An empty rank-local model (after init): set its tensors with shard_tensor() slices, then finalize()."""
    from . import gguf_synth as gs
    m = capi.Model(be, gs.model_config(local_spec(spec, world), max_blocks, max_seqs, max_batch_tokens, max_blocks_per_seq))
    m._ck(m.lib.vx_model_enable_tp(m.h, spec.vocab))
    return m


def load_sharded(be, spec, tensors, rank, world, **cfg):
    """Builds this rank's model from an iterable of whole (layer, slot, type, raw) tensors."""
    m = create_model(be, spec, world, **cfg)
    for layer, slot, t, raw in tensors:
        m.set_tensor(layer, slot, t, shard_tensor(layer, slot, t, raw, rank, world))
    m.finalize()
    return m
