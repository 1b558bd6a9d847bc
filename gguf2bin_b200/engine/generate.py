"""The generation loop: batches of unequal prompts, stop tokens, sequences that end
earlier, and as many batches one after another as there are requests.

The loop follows the reference's ``run`` (src/main.c:320-348 of AnonymoDGH/gguf2bin):
the whole prompt first, then sample / feed until ``-n`` tokens exist or the context is
full (src/main.c:337-340).  Stop tokens follow its ``chat`` (src/main.c:442): a sampled
stop token ends the sequence, is not part of the output and is not fed back.  Unlike the
reference, an over-long prompt is an error instead of being cut (src/main.c:321-324),
and the last sampled token is not fed when nothing will be sampled after it.

All decisions are host code over a small backend interface, so they can be tested
without a device:

    backend.page_size, backend.free_pages, backend.max_context
    backend.open(stream_id, reserve_tokens) -> handle     (a slot and its pages)
    backend.close(handle)                                  (gives them back)
    backend.prefill(handles, prompts) -> first sampled token of each
    backend.decode(handles, tokens)   -> next sampled token of each, after feeding one
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence


class GenerationError(ValueError):
    """A request that cannot be served (empty or over-long prompt, no room at all)."""


@dataclass
class Generation:
    tokens: list = field(default_factory=list)       # generated ids, stop token excluded
    finish_reason: str = ""                          # "stop" | "length" | "context"
    stop_token: Optional[int] = None


def pages_for(tokens: int, page_size: int) -> int:
    return -(-int(tokens) // page_size)


def reserve_tokens(prompt_len: int, max_new: int, max_context: int) -> int:
    """Positions a request can come to hold: its prompt and every generated token that
    is fed back (the last one is not)."""
    return min(max_context, prompt_len + max(0, max_new - 1))


def plan_batch(prompt_lens: Sequence[int], max_new: int, max_context: int, page_size: int,
               free_pages: int, max_batch: int) -> int:
    """How many of the pending requests (in order) start together: as many as fit the
    free pages with room for all they may generate, at most ``max_batch``, at least one."""
    used = n = 0
    for plen in prompt_lens[:max_batch]:
        need = pages_for(reserve_tokens(plen, max_new, max_context), page_size)
        if used + need > free_pages:
            break
        used += need
        n += 1
    if n == 0:
        need = pages_for(reserve_tokens(prompt_lens[0], max_new, max_context), page_size)
        raise GenerationError(f"a request needs {need} pages of {page_size} tokens but the cache "
                              f"has {free_pages} free; enlarge max_tokens")
    return n


def decide(token: int, n_generated: int, prompt_len: int, stop_ids, max_new: int,
           max_context: int) -> tuple[bool, Optional[str]]:
    """After ``token`` was sampled as the ``n_generated``-th new token (1-based):
    (keep the token?, finish reason or None)."""
    if token in stop_ids:
        return False, "stop"
    if n_generated >= max_new:
        return True, "length"
    if prompt_len + n_generated >= max_context:          # no position left to sample from
        return True, "context"
    return True, None


def generate(backend, prompts: Sequence[Sequence[int]], max_new_tokens: int,
             stop_ids=(), max_batch: int = 64, first_stream: int = 0) -> list[Generation]:
    """Generates for every prompt; results come back in the order of the prompts."""
    stop_ids = frozenset(int(s) for s in stop_ids)
    max_context = backend.max_context
    for i, p in enumerate(prompts):
        if len(p) < 1:
            raise GenerationError(f"prompt {i} is empty")
        if len(p) > max_context:
            raise GenerationError(f"prompt {i} has {len(p)} tokens; the context holds {max_context}")
    results = [Generation() for _ in prompts]
    start = 0
    while start < len(prompts):
        pending = [len(p) for p in prompts[start:]]
        k = plan_batch(pending, max_new_tokens, max_context, backend.page_size,
                       backend.free_pages, max_batch)
        idx = list(range(start, start + k))
        start += k
        _run_batch(backend, prompts, idx, results, max_new_tokens, stop_ids, max_context,
                   first_stream)
    return results


def _run_batch(backend, prompts, idx, results, max_new, stop_ids, max_context, first_stream):
    handles = {}
    try:
        for i in idx:
            handles[i] = backend.open(first_stream + i,
                                      reserve_tokens(len(prompts[i]), max_new, max_context))
        live = list(idx)
        if max_new <= 0:
            for i in live:
                results[i].finish_reason = "length"
            live = []
        sampled = {}
        if live:
            first = backend.prefill([handles[i] for i in live], [list(prompts[i]) for i in live])
            sampled = dict(zip(live, first))
        while live:
            still = []
            for i in live:
                plen = len(prompts[i])
                if plen >= max_context and not results[i].tokens:   # src/main.c:337-340
                    results[i].finish_reason = "context"
                    reason = "context"
                else:
                    tok = int(sampled[i])
                    keep, reason = decide(tok, len(results[i].tokens) + 1, plen, stop_ids, max_new,
                                          max_context)
                    if keep:
                        results[i].tokens.append(tok)
                    else:
                        results[i].stop_token = tok
                    if reason:
                        results[i].finish_reason = reason
                if reason:
                    backend.close(handles.pop(i))          # its slot and pages are free again
                else:
                    still.append(i)
            live = still
            if live:
                nxt = backend.decode([handles[i] for i in live],
                                     [results[i].tokens[-1] for i in live])
                sampled = dict(zip(live, nxt))
    finally:
        for h in handles.values():
            backend.close(h)
