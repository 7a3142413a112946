"""Writes the golden fixtures of this folder.

    python tests/golden/make_golden.py

1. flash_attn_kat.json -- the one known-answer test the reference stores for this path:
   inputs are closed-form (arange(48) in bf16 divided by 30/40/50), expected outputs are the
   24+24 literals of rllm/tch-cuda/tests/flash_attn_tests.rs:35-74 (rounded to 4 digits there).
   The literals below were transcribed from that file; they pin the CPU oracle.
2. cache_and_decode_small.npz -- a small seeded case (inputs + expected outputs) for
   reshape_and_cache, gather_cached_kv, copy_blocks and paged attention.  The reference has no
   stored vectors for these; the expected outputs come from the PyTorch-CPU port of
   rllm/rllm-cuda/src/llm/refkernels.rs (oracle/refkernels_cpu.py) and are checked against
   the C oracle when the fixture is written.
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import cpu_oracle, refkernels_cpu  # noqa: E402

KAT_EXPECTED = [
    [[0.084, 0.1035, 0.124, 0.1436, 0.1641, 0.1836, 0.2031, 0.2236],
     [0.0923, 0.1118, 0.1318, 0.1523, 0.1719, 0.1924, 0.2119, 0.2324]],
    [[0.4199, 0.4395, 0.459, 0.4805, 0.5, 0.5195, 0.543, 0.5625],
     [0.4277, 0.4473, 0.4668, 0.4883, 0.5078, 0.5273, 0.5508, 0.5703]],
    [[0.7539, 0.7734, 0.793, 0.8125, 0.832, 0.8516, 0.875, 0.8945],
     [0.7617, 0.7813, 0.8008, 0.8203, 0.8398, 0.8594, 0.8828, 0.9023]],
]


def write_kat():
    kat = {
        "source": "rllm/tch-cuda/tests/flash_attn_tests.rs:35-74",
        "inputs": "q = arange(48, bf16).reshape(3,2,8); k = q/40; v = q/50; q = q/30; "
                  "each transposed to [2 tokens, 3 heads, 8]; cu_seqlens [0,2]; "
                  "max_seqlen 32; softmax_scale 0.5; causal false; output transposed back",
        "round_digits": 4,
        "expected": KAT_EXPECTED,
    }
    with open(os.path.join(HERE, "flash_attn_kat.json"), "w") as f:
        json.dump(kat, f, indent=1)


def digest(t: torch.Tensor) -> str:
    import hashlib
    return hashlib.sha256(t.contiguous().view(torch.int16).numpy().tobytes()).hexdigest()


def small_case(seed=1234):
    g = torch.Generator().manual_seed(seed)
    nblk, hkv, hq, d, bs, x = 12, 2, 8, 128, 16, 8
    kc = torch.randn(nblk, hkv, d // x, bs, x, generator=g).to(torch.bfloat16)
    vc = torch.randn(nblk, hkv, d, bs, generator=g).to(torch.bfloat16)
    ctx = [1, 17, 40, 16]
    tables = [[3], [7, 1], [5, 0, 9], [2]]
    bt = torch.zeros(len(ctx), 3, dtype=torch.int32)
    for i, r in enumerate(tables):
        bt[i, :len(r)] = torch.tensor(r, dtype=torch.int32)
    q = torch.randn(len(ctx), hq, d, generator=g).to(torch.bfloat16)
    nk = torch.randn(len(ctx), hkv, d, generator=g).to(torch.bfloat16)
    nv = torch.randn(len(ctx), hkv, d, generator=g).to(torch.bfloat16)
    slots = torch.tensor([tables[i][(c - 1) // bs] * bs + (c - 1) % bs for i, c in enumerate(ctx)],
                         dtype=torch.int32)
    return dict(kc=kc, vc=vc, ctx=torch.tensor(ctx, dtype=torch.int32), bt=bt, q=q, nk=nk, nv=nv,
                slots=slots, hkv=hkv, hq=hq, bs=bs)


def write_small():
    c = small_case()
    kc, vc = c["kc"].clone(), c["vc"].clone()
    refkernels_cpu.reshape_and_cache(c["nk"], c["nv"], kc, vc, c["slots"])
    kc2, vc2 = c["kc"].clone(), c["vc"].clone()
    cpu_oracle.reshape_and_cache(c["nk"], c["nv"], kc2, vc2, c["slots"])
    assert torch.equal(kc.view(torch.int16), kc2.view(torch.int16))
    assert torch.equal(vc.view(torch.int16), vc2.view(torch.int16))
    scale = refkernels_cpu.default_scale(128)
    dec = refkernels_cpu.decode_step_cpu(c["q"].float(), kc.float(), vc.float(), c["hkv"], scale,
                                         c["bt"], c["ctx"], c["bs"])
    dec2 = cpu_oracle.paged_attention_v1(c["q"], kc, vc, c["hkv"], scale, c["bt"], c["ctx"])
    assert (dec - dec2).abs().max() < 2e-5, float((dec - dec2).abs().max())
    # fork: block 3 -> 10, 11 ; block 9 -> 4
    mapping = [3, 10, 3, 11, 9, 4]
    kcf, vcf = kc.clone(), vc.clone()
    cpu_oracle.copy_blocks([kcf], [vcf], mapping)
    # caches are stored as SHA-256 digests of their bf16 bit patterns (bit-exact checks only
    # need equality); the decode output is stored as values
    np.savez_compressed(
        os.path.join(HERE, "cache_and_decode_small.npz"),
        decode_out=dec.numpy(), block_mapping=np.array(mapping, dtype=np.int64),
        digests=np.array([digest(kc), digest(vc), digest(kcf), digest(vcf)]))


if __name__ == "__main__":
    write_kat()
    write_small()
    print("golden fixtures written to", HERE)
