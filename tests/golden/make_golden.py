"""Generates ``tests/golden/config1_layer_step.npz``: known-answer vectors for one
layer-step of configuration 1 (OPT-125m shapes, fp32, 8 requests, CPU-sized).

The reference ships no golden vectors for this path and cannot be imported here
(it needs vLLM 0.5.0.post1 and a GPU), so these vectors are produced by the CPU oracle
(``oracle/hybrid_cache_oracle.py``) from a seeded workload.  They pin the oracle and the
workload generator against drift, and give the GPU kernels a fixed target.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from apt_serve_b200.workloads import make_config_workload  # noqa: E402
from oracle import hybrid_cache_oracle as O  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config1_layer_step.npz")


def build():
    w = make_config_workload(1, kv_from_projection=True)
    wk, bk, wv, bv = w.kv_weights()
    cache = w.kv_cache.clone()
    out = O.decode_layer_step(w.hidden_states, w.query, w.new_key, w.new_value, cache, cache, wk, bk,
                              wv, bv, w.meta, w.scale)
    m = w.meta
    new_slots = m.slot_mapping[m.hidden_holder_upd]
    rows = O.flat_rows(cache)
    return {
        "seq_lens": np.asarray(w.seq_lens, dtype=np.int32),
        "use_hidden": np.asarray(w.use_hidden, dtype=np.bool_),
        "slot_mapping_head": m.slot_mapping[:64].numpy(),
        "private_block_tables": m.private_block_tables.numpy(),
        "new_token_slots": new_slots.numpy(),
        "attention_output": out.numpy().astype(np.float32),
        # checksums: the cache before the step, after it, and the rows the step wrote
        # (sums of magnitudes: the K/V blocks hold CPU matrix products, whose last bits depend
        # on the machine's BLAS, so the tests compare these to 1e-6 and not bit for bit)
        "cache_sum_before": np.float64(w.kv_cache.double().abs().sum().item()),
        "cache_sum_after": np.float64(cache.double().abs().sum().item()),
        "written_rows": rows[new_slots[torch.tensor(w.use_hidden)]][:, :8].numpy().astype(np.float32),
    }


if __name__ == "__main__":
    np.savez_compressed(OUT, **build())
    print(OUT, os.path.getsize(OUT), "bytes")
