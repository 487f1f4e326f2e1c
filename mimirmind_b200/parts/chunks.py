"""A step's tokens cut into chunks of a fixed number of tokens, per request in order: what the scans over long portions
(the minGRU's, the matrix-state mixers') walk side by side.  Made once per step on the host and shared by the layers."""
from __future__ import annotations

import numpy as np
import torch

from .base import StepContext


def token_chunks(ctx: StepContext, chunk: int):
    """(chunk_meta int32 [chunks, 4] = (first token, tokens, request, first chunk of its request ? 1 : 0),
    req_chunks int32 [requests, 2] = (first chunk, chunks)), both on the device."""
    key = ("token_chunks", chunk)
    if key not in ctx.derived:
        meta, per_req = [], []
        for r, (s, n) in enumerate(zip(ctx.q_start, ctx.q_len)):
            first = len(meta)
            for off in range(0, n, chunk):
                meta.append((s + off, min(chunk, n - off), r, int(off == 0)))
            per_req.append((first, len(meta) - first))
        host = np.concatenate([np.asarray(meta, dtype=np.int32).reshape(-1), np.asarray(per_req, dtype=np.int32).reshape(-1)])
        # from pinned memory, without waiting for the device (a pageable copy would stall the launches behind it)
        pinned = torch.from_numpy(host).pin_memory()
        dev = pinned.to(ctx.token_ids.device, non_blocking=True)
        ctx.derived[key] = (dev[:4 * len(meta)].view(len(meta), 4), dev[4 * len(meta):].view(len(per_req), 2))
        ctx.derived[key + ("staged",)] = pinned
    return ctx.derived[key]
