"""CPU point of the decode benchmark: the Llama-3-8B-shaped W8A8 decoder on the host CPUs, every linear on the host
runtime's pinned worker pools (AMX int8 / AVX-512 VNNI), random int8 weights, one sequence.  No GPU needed.

python benchmarks/bench_host_decode.py [--layers 32] [--prompt-len 1024] [--new 8]
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.hostrt.host_model import HostDecoder  # noqa: E402
from mojo_linuxperiments_b200.models import config as C  # noqa: E402


def random_checkpoint(cfg, seed=0):
    """int8 weights uniform[-127,127] + scales chosen so that activations keep unit scale; checkpoint-dict layout."""
    g = torch.Generator().manual_seed(seed)
    d, hd = cfg.d_model, cfg.head_dim

    def lin(n, k):
        return (torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8),
                torch.full((n,), 1.0 / (73.0 * k ** 0.5), dtype=torch.float32))
    ck = {"embed": torch.randn((cfg.vocab, d), generator=g).to(torch.bfloat16), "final_norm": torch.ones(d, dtype=torch.bfloat16)}
    ck["lm_head.qweight"], ck["lm_head.scale"] = lin(cfg.vocab, d)
    for l in range(cfg.n_layers):
        p = f"layers.{l}."
        ck[p + "attn_norm"] = torch.ones(d, dtype=torch.bfloat16)
        ck[p + "mlp_norm"] = torch.ones(d, dtype=torch.bfloat16)
        for name, n, k in (("wq", cfg.n_heads * hd, d), ("wk", cfg.n_kv_heads * hd, d), ("wv", cfg.n_kv_heads * hd, d),
                           ("wo", d, cfg.n_heads * hd), ("gate", cfg.ffn, d), ("up", cfg.ffn, d), ("down", d, cfg.ffn)):
            ck[p + name + ".qweight"], ck[p + name + ".scale"] = lin(n, k)
    return ck


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--new", type=int, default=8)
    ap.add_argument("--isa", default="best")
    a = ap.parse_args()
    from dataclasses import replace
    cfg = replace(C.llama3_8b(), n_layers=a.layers)
    t0 = time.monotonic()
    ck = random_checkpoint(cfg)
    dec = HostDecoder(cfg, ck, isa=a.isa)
    t_init = time.monotonic() - t0
    prompt = torch.randint(0, cfg.vocab, (a.prompt_len,), generator=torch.Generator().manual_seed(1))
    t0 = time.monotonic()
    lg = dec.forward(prompt)
    ttft = time.monotonic() - t0
    lin_prefill = dec.linear_ns * 1e-9
    dec.linear_ns = 0
    t0 = time.monotonic()
    for _ in range(a.new):
        lg = dec.forward(torch.tensor([int(lg.argmax())]))
    per_tok = (time.monotonic() - t0) / a.new
    print(json.dumps({"op": "host decode, llama3-8b shape", "layers": a.layers, "full_model": a.layers == 32,
                      "prompt_len": a.prompt_len, "ttft_s": ttft, "ttft_linear_s": lin_prefill,
                      "decode_s_per_token_bs1": per_tok, "decode_linear_s_per_token": dec.linear_ns * 1e-9 / a.new,
                      "tokens_per_s_bs1": 1.0 / per_tok, "weights_init_s": t_init}), flush=True)


if __name__ == "__main__":
    main()
