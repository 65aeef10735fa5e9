"""Sequence-length sweep of the MTA module that writes the reference's benchmark records.

    python -m multitokenatention_triton_b200.benchmark_seq_len [--start 128 --end 1024 --step 128] [--out results.jsonl]

One JSON object per line with the keys of the reference's sweep (benchmark_seq_len.py:172-189) so that its plotting
script reads the file unchanged: seq_len, batch_size, n_heads, head_dim, dropout, causal, dtype, use_mask, the four
kernel sizes, and the times in milliseconds.  `triton_fwd_time` / `triton_bwd_time` are this library's module
(forward under no_grad = the fused forward; forward + backward through the stage-by-stage path); `pytorch_fwd_time` /
`pytorch_bwd_time` are a plain PyTorch evaluation of the same pipeline on the same GPU (mask, pad, conv2d, linear,
softmax as in mta_attention_pytorch.py:56-112), None when it does not fit in memory.
"""
import argparse
import json
import time
import types

import torch
import torch.nn.functional as F

from . import MTAAttentionTriton


def torch_mta_forward(q, k, v, w1, W1, w2, W2):
    """The reference's PyTorch pipeline (mta_attention_pytorch.py:56-112) with a causal mask."""
    S = q.size(-2)
    mask = torch.triu(torch.full((S, S), float("-inf"), device=q.device, dtype=q.dtype), diagonal=1)
    dead = mask == float("-inf")
    s = torch.matmul(q, k.transpose(2, 3)) * q.size(-1) ** -0.5

    def conv(x, w):
        x = torch.where(dead, 0.0, x)
        x = F.pad(x, ((w.size(-1) - 1) // 2, (w.size(-1) - 1) // 2, w.size(-2) - 1, 0), value=0.0)
        return F.conv2d(x, w.unsqueeze(1), padding=0, groups=x.size(1))

    s = conv(s, w1)
    s = F.linear(s.transpose(1, -1), W1).transpose(1, -1)
    s = F.softmax((s + mask).float(), dim=-1).type_as(q)
    s = torch.where(dead, 0.0, conv(s, w2))
    s = F.linear(s.transpose(1, -1), W2).transpose(1, -1)
    return torch.matmul(s, v).transpose(1, 2)


def _time(fn, warmup, runs):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(runs):
        fn()
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) * 1e3 / runs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--start", type=int, default=128)
    ap.add_argument("--end", type=int, default=1024)
    ap.add_argument("--step", type=int, default=128)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--runs", type=int, default=10)
    ap.add_argument("--out", default="benchmark_results.jsonl")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    dtype = getattr(torch, a.dtype)
    cfg = types.SimpleNamespace(use_mta=True, query_kernel_size=6, key_kernel_size=11, after_sm_query_kernel_size=6,
                                after_sm_key_kernel_size=11, pre_sm_linear_head=True, post_sm_linear_head=True,
                                pad_key="both", init_method="identity", dim=a.heads * a.dim)
    with open(a.out, "w") as fh:
        for S in range(a.start, a.end + 1, a.step):
            m = MTAAttentionTriton(a.heads, cfg, dropout=0.0, causal=True).to(dev).to(dtype).eval()
            m.reset_mta_parameters()
            torch.manual_seed(123)
            q, k, v = (torch.randn(a.batch, a.heads, S, a.dim, device=dev, dtype=dtype, requires_grad=True) for _ in range(3))
            w = [m.mta_conv_triton.weight, m.wpsm_triton.weight, m.mta_conv_after_sm_triton.weight, m.wposm_triton.weight]

            def ours_fwd():
                with torch.no_grad():
                    m(q, k, v, None, None)

            def ours_bwd():
                m(q, k, v, None, None).sum().backward()

            def torch_fwd():
                with torch.no_grad():
                    torch_mta_forward(q, k, v, *w)

            def torch_bwd():
                torch_mta_forward(q, k, v, *w).sum().backward()

            rec = {"seq_len": S, "batch_size": a.batch, "n_heads": a.heads, "head_dim": a.dim, "dropout": 0.0, "causal": True,
                   "dtype": str(dtype), "use_mask": False, "query_kernel_size": 6, "key_kernel_size": 11,
                   "after_sm_query_kernel_size": 6, "after_sm_key_kernel_size": 11}
            for key, fn in (("pytorch_fwd_time", torch_fwd), ("triton_fwd_time", ours_fwd), ("pytorch_bwd_time", torch_bwd),
                            ("triton_bwd_time", ours_bwd)):
                try:
                    rec[key] = _time(fn, a.warmup, a.runs)
                except torch.cuda.OutOfMemoryError:
                    rec[key] = None
                    torch.cuda.empty_cache()
            fh.write(json.dumps(rec) + "\n")
            fh.flush()
            print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
