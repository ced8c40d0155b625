"""Small, self-ending cases for `ncu` captures of the library's kernels.

    python open-vc-attention_b200/profile_case.py attention --seq 16384 --heads 9   # FP8 inputs prepared once, 3 attention launches
    python open-vc-attention_b200/profile_case.py call --seq 73397 --heads 7        # 2 complete attention(q, k, v) calls (4 launches each)

Inputs are i.i.d. N(0,1) BF16 on cuda:0 from a fixed seed.  Run the same command once without ncu first.
"""

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from open_vc_attn import api, forward, preparation  # noqa: E402


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("case", choices=["attention", "call"])
    parser.add_argument("--seq", type=int, default=16384)
    parser.add_argument("--heads", type=int, default=9)
    args = parser.parse_args()
    torch.manual_seed(0)
    q, k, v = [torch.randn(args.seq, args.heads, 128, device="cuda:0", dtype=torch.bfloat16) for _ in range(3)]
    if args.case == "attention":
        prepared = preparation._prepare_packed(q, k, v, tuple(q.shape))
        for _ in range(3):
            out = api.attention_fp8(prepared)
    else:
        for _ in range(2):
            out = api.attention(q, k, v)
    torch.cuda.synchronize()
    forward.check_status(q.device)
    print("mean |out|", float(out.float().abs().mean()))


if __name__ == "__main__":
    main()
