#!/usr/bin/env python
"""Small single-GPU workload for profiling the tcgen05 attention kernel: a few launches on batch 8 x seq 2048 x 4 heads
(48 MB of qkv).  Run it plainly first, then under ncu as described in profiles/attention_fwd_b8_s2048_h4.md."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import torch  # noqa: E402

from iris_b200.ops.attention import attention_fwd  # noqa: E402


def main():
    batch, seq, heads = 8, 2048, 4
    g = torch.Generator(device="cuda").manual_seed(1)
    qkv = torch.randn((batch * seq, 3 * heads * 128), generator=g, device="cuda").to(torch.bfloat16)
    out = torch.empty((batch * seq, heads * 128), dtype=torch.bfloat16, device="cuda")
    for _ in range(4):
        attention_fwd(qkv, out, batch, seq, heads)
    torch.cuda.synchronize()
    print("attention profile workload done", float(out.float().abs().mean()))


if __name__ == "__main__":
    main()
