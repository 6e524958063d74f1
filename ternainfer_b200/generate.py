"""Greedy generation driver around the TernaSpMM model (``FastGen``).

Mirrors ``generate.py`` of Gu-J/TernaInfer in what matters for the hot path:
the prefill forward and the one-token decode forward are each captured into a
CUDA graph after a warm-up forward (:121-154, :192-224) and replayed with
static input tensors, greedy sampling is an argmax over the logits of each
sequence's last position (:274, :283, :305) - taken inside the output-head
kernel, so the graphs return token ids - and throughput is reported per phase.  Tokenizer, chat format and top-p
sampling of the reference are not rebuilt: prompts are token ids.
"""
from __future__ import annotations

import argparse
import time
from dataclasses import dataclass

import torch

from .model import ModelArgs, Transformer


@dataclass
class GenArgs:
    gen_length: int = 128
    gen_bsz: int = 1
    prompt_length: int = 512
    use_cuda_graph: bool = True


class FastGen:
    def __init__(self, model: Transformer, gen_args: GenArgs, device="cuda"):
        self.model, self.args, self.device = model, gen_args, torch.device(device)
        a = gen_args
        assert a.prompt_length + a.gen_length <= model.max_seq_len
        self.cache = model.make_cache(a.gen_bsz, self.device)
        self._prefill_tokens = torch.zeros((a.gen_bsz, a.prompt_length), dtype=torch.long, device=self.device)
        self._prefill_pos = torch.arange(a.prompt_length, device=self.device)
        self._tokens = torch.zeros((a.gen_bsz, 1), dtype=torch.long, device=self.device)
        self._pos = torch.zeros(1, dtype=torch.long, device=self.device)
        self._prefill_graph = self._decode_graph = None
        self._prefill_next = self._decode_next = None

    @torch.inference_mode()
    def _capture(self):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):          # warm-up forwards outside capture (one-time library set-up)
            self.model(self._prefill_tokens, self.cache, self._prefill_pos, greedy_last=True)
            self.model(self._tokens, self.cache, self._pos, greedy_last=True)
        torch.cuda.current_stream().wait_stream(s)
        self._prefill_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._prefill_graph):
            self._prefill_next = self.model(self._prefill_tokens, self.cache, self._prefill_pos, greedy_last=True)
        self._decode_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._decode_graph):
            self._decode_next = self.model(self._tokens, self.cache, self._pos, greedy_last=True)

    @torch.inference_mode()
    def generate(self, prompt: torch.Tensor):
        """prompt [B, prompt_length] token ids -> (tokens [B, gen_length], stats)."""
        a = self.args
        if a.use_cuda_graph and self._decode_graph is None:
            self._capture()
        out = torch.empty((a.gen_bsz, a.gen_length), dtype=torch.long, device=self.device)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        self._prefill_tokens.copy_(prompt)
        if a.use_cuda_graph:
            self._prefill_graph.replay()
            nxt = self._prefill_next
        else:
            nxt = self.model(self._prefill_tokens, self.cache, self._prefill_pos, greedy_last=True)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        for i in range(a.gen_length):
            out[:, i] = nxt
            if i == a.gen_length - 1:
                break
            self._tokens.copy_(nxt[:, None])
            self._pos.fill_(a.prompt_length + i)
            if a.use_cuda_graph:
                self._decode_graph.replay()
                nxt = self._decode_next
            else:
                nxt = self.model(self._tokens, self.cache, self._pos, greedy_last=True)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        stats = {"prefill_s": t1 - t0, "decode_s": t2 - t1,
                 "prefill_tokens_per_s": a.gen_bsz * a.prompt_length / (t1 - t0),
                 "decode_tokens_per_s": a.gen_bsz * (a.gen_length - 1) / (t2 - t1)}
        return out, stats


def build_random_model(args: ModelArgs, max_seq_len: int, seed: int = 1234, dense: bool = False):
    from .convert.convert_TernaInfer import random_checkpoint
    dic = random_checkpoint(args.dim, args.n_layers, args.n_heads, args.n_kv_heads, args.ffn_dim, args.vocab_size,
                            seed=seed, dense=dense)
    with torch.device("cuda"):
        model = Transformer(args, dic, max_seq_len=max_seq_len)
    return model.cuda().to(torch.bfloat16), dic


def main():
    ap = argparse.ArgumentParser(description="greedy decode of a random-init BitNet-style model")
    ap.add_argument("--layers", type=int, default=30)
    ap.add_argument("--bsz", type=int, default=1)
    ap.add_argument("--prompt_length", type=int, default=512)
    ap.add_argument("--gen_length", type=int, default=128)
    ap.add_argument("--no_cuda_graph", action="store_true")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--fused_glue", action="store_true", help="fused norm+quantiser kernels, residual add in the epilogue")
    a = ap.parse_args()
    margs = ModelArgs(n_layers=a.layers, fused_glue=a.fused_glue)
    model, _ = build_random_model(margs, a.prompt_length + a.gen_length, a.seed)
    gen = FastGen(model, GenArgs(a.gen_length, a.bsz, a.prompt_length, not a.no_cuda_graph))
    g = torch.Generator(device="cuda").manual_seed(a.seed + 1)
    prompt = torch.randint(0, margs.vocab_size, (a.bsz, a.prompt_length), generator=g, device="cuda")
    gen.generate(prompt)            # warm-up (captures the graphs)
    tokens, stats = gen.generate(prompt)
    print({k: round(v, 4) for k, v in stats.items()}, "first tokens", tokens[0, :8].tolist())


if __name__ == "__main__":
    main()
