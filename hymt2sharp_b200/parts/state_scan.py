"""What mixers with a matrix of state per head share: how a step's tokens are cut into chunks for the three-pass form of
their recurrence (kernels.ops.linear_scan).  A helper of mixers, not a part category of its own."""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops


def chunk_plan(ctx):
    """None for a step that runs serially (decode steps, short portions); else (count, chunk_seq, chunk_first, chunk_len,
    seq_chunk0) on the device: every sequence's new tokens in consecutive chunks of a fixed size, the last one shorter.
    Worked out once per step and kept in `ctx.shared` for every layer that scans."""
    key = "linear_scan_chunks"
    if key in ctx.shared:
        return ctx.shared[key]
    chunk, minimum = ops.linear_scan_chunking()
    plan = None
    if ctx.max_new_tokens >= minimum and ctx.host_new_tokens:
        news = np.asarray(ctx.host_new_tokens, dtype=np.int64)
        firsts = np.concatenate([[0], np.cumsum(news)[:-1]])
        per = -(-news // chunk)
        seq0 = np.concatenate([[0], np.cumsum(per)])
        count = int(seq0[-1])
        cseq = np.repeat(np.arange(len(news)), per)
        within = np.arange(count) - seq0[cseq]
        cfirst = firsts[cseq] + within * chunk
        clen = np.minimum(chunk, news[cseq] - within * chunk)
        flat = np.concatenate([cseq, cfirst, clen, seq0]).astype(np.int32)
        dev = torch.from_numpy(flat).to(ctx.device, non_blocking=True)
        plan = (count, dev[:count], dev[count:2 * count], dev[2 * count:3 * count], dev[3 * count:])
    ctx.shared[key] = plan
    return plan
