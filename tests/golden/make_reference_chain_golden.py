"""Generates ``tests/golden/reference_chain_decode.npz``: outputs of the REFERENCE's own decode
op chain, run on a B200 with the kernels the reference runs -- its ``mixed_cache.cu``
compiled unmodified (``oracle/_ref``), ``torch.nn.functional.linear`` (cuBLAS) for the
``kv_only`` projection, vLLM's ``reshape_and_cache_flash`` and flash-attention paged
decode (aptserve_opt.py:106-124, aptserve_flash_attn.py:356-387, 452-473).

The inputs are seeded workloads that the CPU can rebuild bit for bit, so the file holds only
the cases' parameters and the chain's outputs.  ``tests/test_golden.py`` checks the CPU
oracle against them without a GPU.  Needs a GPU, the built ``oracle/_ref`` extension and
vLLM's flash-attention; run from the repository root:

    python tests/golden/make_reference_chain_golden.py [output.npz]
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from apt_serve_b200.workloads import LayerShape, make_decode_workload  # noqa: E402
from oracle.literal_chain_gpu import LiteralChain  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_chain_decode.npz")

# name -> (heads, head size, hidden size, sequence lengths, hidden-cached flags, seed, projected K/V cache)
CASES = {
    # every request hidden-cached: gather, GEMM, scatter into the shared cache, paged attention
    "all_hidden": (4, 128, 512, [5, 129, 300, 16, 1, 700], [True] * 6, 33, False),
    # a mixed batch inside the envelope where the reference's mixed_kv_to_cache index is the
    # intended one (hidden tokens <= 2 x K/V requests)
    "mixed": (4, 128, 512, [30, 17, 33] + [int(x) for x in np.random.default_rng(1).integers(1, 400, size=40)],
              [True] * 3 + [False] * 40, 21, True),
    # K/V-cached requests only: the private cache through the third-party paged attention
    "kv_only": (4, 128, 512, [1, 15, 16, 17, 127, 128, 129, 300, 1000, 2048], [False] * 10, 5, False),
}


def build_case(case):
    """The case's workload, drawn on the CPU (the random stream of a CUDA generator differs)."""
    heads, d, e, lens, hid, seed, proj = CASES[case]
    shape = LayerShape("golden", heads, d, e, torch.float16)
    return make_decode_workload(shape, list(lens), list(hid), seed=seed, device="cpu",
                                with_shared_cache=any(hid), kv_from_projection=proj)


# The three mixed_cache_ops of the reference build on their own, bit for bit.  "outside": more
# hidden tokens than twice the K/V requests, where the kernel's `blockIdx.x % (2 * n_kv)` index
# (mixed_cache.cu:88) re-reads the first 2 * n_kv hidden tokens instead of walking all of them
# (every index it forms stays inside its tensor as long as there is at least one K/V request).
OPS_CASES = {
    "ops_inside": ([3, 40, 17, 4, 64, 9], [True, False, False, True, False, False]),
    "ops_outside": ([3, 40, 17, 4, 64, 9], [True, True, False, True, False, True]),
}


def build_ops_case(case):
    lens, hid = OPS_CASES[case]
    shape = LayerShape("golden-ops", 1, 32, 32, torch.float16)
    w = make_decode_workload(shape, lens, hid, seed=3, device="cpu", with_shared_cache=True)
    g = torch.Generator().manual_seed(1)
    n = w.meta.num_tot_tokens
    key = torch.randn(n, 1, 32, generator=g).to(torch.float16)
    value = torch.randn(n, 1, 32, generator=g).to(torch.float16)
    holder = torch.randn(n, 32, generator=g).to(torch.float16)
    return w, key, value, holder


def record_ops(out):
    from oracle import build_ref
    ext = build_ref.load()
    for case in OPS_CASES:
        w, key, value, holder = build_ops_case(case)
        assert w.meta.kv_cache_use_tot.numel() > 0
        d, m = w.to("cuda"), None
        m = d.meta
        hold = holder.cuda()
        ext.hidden_to_cache(d.hidden_states, d.kv_cache, m.slot_mapping, m.hidden_cache_use_input,
                            m.hidden_cache_store_tot)
        torch.cuda.synchronize()
        ext.cache_to_hidden(hold, d.kv_cache, m.slot_mapping, m.hidden_cache_use_tot)
        torch.cuda.synchronize()
        ext.mixed_kv_to_cache(key.cuda(), value.cuda(), d.kv_cache[0], d.kv_cache[1], d.shared_cache[0],
                              d.shared_cache[1], m.slot_mapping, m.slot_mapping_shared, m.kv_cache_use_tot,
                              m.hidden_cache_use_tot)
        torch.cuda.synchronize()
        out[case + "/kv_cache"] = d.kv_cache.cpu().numpy().view(np.uint16)
        out[case + "/shared_cache"] = d.shared_cache.cpu().numpy().view(np.uint16)
        out[case + "/hidden_holder"] = hold.cpu().numpy().view(np.uint16)


def build_cache_write_case():
    """Inputs of the recorded `reshape_and_cache_flash` call: strided key / value rows (views
    of a fused QKV tensor, as in the model), slots in random order, some of them -1."""
    g = torch.Generator().manual_seed(7)
    heads, d, bs, nb, t = 2, 32, 16, 12, 50
    qkv = torch.randn(t, 3 * heads * d, generator=g).to(torch.float16)
    key = qkv[:, heads * d:2 * heads * d].view(t, heads, d)
    value = qkv[:, 2 * heads * d:].view(t, heads, d)
    slots = torch.randperm(nb * bs, generator=g)[:t].to(torch.int64)
    slots[::7] = -1
    cache = torch.randn(2, nb, bs, heads, d, generator=g).to(torch.float16)
    return key, value, slots, cache


def record_cache_write(out, chain):
    key, value, slots, cache = build_cache_write_case()
    c = cache.cuda()
    chain.reshape_and_cache(key.cuda(), value.cuda(), c[0], c[1], slots.cuda())
    torch.cuda.synchronize()
    out["reshape_and_cache_flash/cache"] = c.cpu().numpy().view(np.uint16)


def main(path):
    chain, why = LiteralChain.create()
    if chain is None:
        raise SystemExit(f"reference chain unavailable: {why}")
    out = {}
    record_ops(out)
    record_cache_write(out, chain)
    for case in CASES:
        w = build_case(case).to("cuda")
        if any(w.use_hidden):
            hd = w.heads * w.shape.head_dim
            y = chain.hybrid_decode_layer(w.hidden_states, w.query, w.qkv_weight[hd:], w.qkv_bias[hd:],
                                          w.kv_cache, w.shared_cache, w.meta, w.scale)
            m = w.meta
            slots = m.slot_mapping[m.hidden_cache_store_tot]
            rows = w.kv_cache.view(-1, w.kv_cache.stride(2))[slots]
            out[case + "/new_hidden_rows"] = rows.cpu().numpy().view(np.uint16)
        else:
            y = chain.decode_attention(w.query, w.kv_cache[0], w.kv_cache[1], w.meta.block_tables,
                                       w.meta.seq_lens_tensor, w.scale)
        torch.cuda.synchronize()
        out[case + "/out"] = y.cpu().numpy().view(np.uint16)      # fp16 bits
        out[case + "/seq_lens"] = np.asarray(w.seq_lens, dtype=np.int32)
    out["attention_name"] = np.asarray(chain.attention_name)
    out["gpu"] = np.asarray(torch.cuda.get_device_name(0))
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else OUT)
