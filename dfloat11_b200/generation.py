"""Greedy generation with the host taken out of the loop: one CUDA graph per single-token step.

The reference measures generation through Hugging Face ``generate`` (inference.py:45-95), where
every token pays the Python cost of a whole forward pass -- some 30 ms for a 36-layer model,
several times what the GPU needs.  Here the single-token step (forward over a static KV cache,
arg-max, position update) is captured once into a CUDA graph and replayed per token.  The DF11
decode hooks run at capture time; their launches through the C ABI are recorded like any other
kernel, so a replay decompresses (or, with ``DF11_FUSED_GEMV=1``, multiplies straight from the
compressed weights) exactly as an eager step would.

Works for any ``transformers`` causal LM whose forward accepts ``past_key_values`` /
``cache_position`` with a ``StaticCache`` -- compressed or not, whole or tensor-parallel (every
rank runs the same loop; the collectives of the partitioned mode are captured with the rest).
Prompts of one batch have the same length; the graph is captured per batch size.
"""
from __future__ import annotations

from typing import Optional

import torch


class GraphedGreedyDecoder:
    """``decoder = GraphedGreedyDecoder(model, max_cache_len=4096); ids = decoder.generate(prompt, 256)``"""

    def __init__(self, model, max_cache_len: int = 4096):
        self.model = model
        self.max_cache_len = int(max_cache_len)
        self.device = next(model.parameters()).device
        if self.device.type != "cuda":
            raise RuntimeError("GraphedGreedyDecoder needs the model on a CUDA device")
        import inspect
        try:
            self._keeps_logits = "logits_to_keep" in inspect.signature(model.forward).parameters
        except (TypeError, ValueError):
            self._keeps_logits = False
        self._cache = None
        self._graph = None
        self._tok = self._pos = self._count = self._produced = None

    # -- one single-token step on static tensors -------------------------------------------------
    def _step(self):
        self._produced.index_copy_(0, self._count, self._tok.view(1, -1))
        logits = self.model(input_ids=self._tok, past_key_values=self._cache, cache_position=self._pos,
                            use_cache=True).logits
        self._tok.copy_(logits[:, -1:].argmax(-1))
        self._pos.add_(1)
        self._count.add_(1)

    def _prepare(self, batch: int):
        from transformers import StaticCache
        dev = self.device
        if self._cache is None or self._tok.shape[0] != batch:
            self._graph = None                            # static tensors change: the old capture is void
            self._cache = StaticCache(config=self.model.config, max_cache_len=self.max_cache_len)
            self._tok = torch.zeros(batch, 1, dtype=torch.int64, device=dev)
            self._pos = torch.zeros(1, dtype=torch.int64, device=dev)
            self._count = torch.zeros(1, dtype=torch.int64, device=dev)
            self._produced = torch.zeros(self.max_cache_len + 8, batch, dtype=torch.int64, device=dev)
        else:
            self._cache.reset()

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int, eos_token_id: Optional[int] = None,
                 eos_check_every: int = 32) -> torch.Tensor:
        """Prompts ``[b, n]`` -> ``[b, n + new]`` ids, greedy.  With one sequence, stops early at
        ``eos_token_id`` (looked for every ``eos_check_every`` tokens, the only host synchronisation
        in the loop)."""
        if input_ids.dim() != 2 or input_ids.shape[0] < 1:
            raise ValueError("input_ids must be [batch, n]")
        if eos_token_id is not None and input_ids.shape[0] != 1:
            raise ValueError("early stopping at an end-of-sequence id is for one sequence at a time")
        n_prompt = input_ids.shape[1]
        if n_prompt + max_new_tokens > self.max_cache_len:
            raise ValueError(f"{n_prompt} + {max_new_tokens} tokens exceed max_cache_len = {self.max_cache_len}")
        if max_new_tokens <= 0:
            return input_ids
        dev = self.device
        input_ids = input_ids.to(dev)
        self._prepare(input_ids.shape[0])
        # only the last position's logits are needed: models whose forward can skip the others
        # (`logits_to_keep`) do not multiply the whole prompt with the output head
        extra = {"logits_to_keep": 1} if self._keeps_logits else {}
        logits = self.model(input_ids=input_ids, past_key_values=self._cache,
                            cache_position=torch.arange(n_prompt, device=dev), use_cache=True, **extra).logits
        self._tok.copy_(logits[:, -1:].argmax(-1))
        self._pos.fill_(n_prompt)
        self._count.zero_()

        steps = max_new_tokens - 1                         # the prefill gave the first new token
        done = 0
        if self._graph is None and steps > 0:
            # two eager steps on a side stream (allocations, lazy initialisation, the hooks' one-time
            # work) advance the generation like any other step; the capture records a step
            # without running it
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                while done < min(2, steps):
                    self._step()
                    done += 1
            torch.cuda.current_stream(dev).wait_stream(side)
            if done < steps:
                torch.cuda.synchronize(dev)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    self._step()
                self._graph = graph
        while done < steps:
            self._graph.replay()
            done += 1
            if eos_token_id is not None and done % eos_check_every == 0:
                if bool((self._produced[:done, 0] == eos_token_id).any()):
                    break
        # the token of the last step is still in `tok`
        self._produced.index_copy_(0, self._count, self._tok.view(1, -1))
        new = self._produced[:done + 1]
        if eos_token_id is not None:
            hit = (new[:, 0] == eos_token_id).nonzero()
            if hit.numel():
                new = new[:int(hit[0]) + 1]
        return torch.cat([input_ids, new.t()], dim=1)

    def reset(self) -> None:
        """Forget the captured graph (after changing the model or the DF11 environment switches)."""
        self._graph = None
