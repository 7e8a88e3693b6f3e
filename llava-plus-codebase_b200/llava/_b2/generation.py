"""Host side of generation that every model of this package shares: the pool of caches that gives each generate() call
one of its own, and the loop that reads tokens from the device's host ring while the device runs ahead."""
import threading

import torch


class _KVPool:
    """KV caches of one engine. Every generate() works on a cache of its own for its whole duration — the reference's
    model_worker runs up to `limit_model_concurrency` generate() threads on one model object
    (llava/serve/model_worker.py:174-185, :230-243), and a shared cache would let request B's prefill overwrite request
    A's context mid-decode. Caches are created on demand (up to `cap`, then acquire() blocks) and reused."""

    def __init__(self, engine, max_batch, max_seq, cap):
        self.engine, self.max_batch, self.max_seq, self.cap = engine, max_batch, max_seq, max(1, int(cap))
        self._cond = threading.Condition()
        self._free, self._made = [], 0

    def acquire(self):
        with self._cond:
            while not self._free and self._made >= self.cap:
                self._cond.wait()
            if self._free:
                return self._free.pop()
            self._made += 1
        try:
            return self.engine.new_kv(self.max_batch, self.max_seq)
        except Exception:
            with self._cond:
                self._made -= 1
                self._cond.notify()
            raise

    def release(self, kv):
        with self._cond:
            self._free.append(kv)
            self._cond.notify()


def _stream_decode(engine, kv, logits, sampling, B, max_new_tokens, eos_ids, pad, prompt, streamer, stopping_criteria,
                   run_ahead=8, begun=False):
    """Host half of the decode loop. The device chooses token 0 from the prefill `logits` and then runs up to `run_ahead`
    steps in front of this loop; `engine.stream_wait(kv, t, B)` hands over token t as soon as its kernel has written it
    to pinned memory. Per token, in the order HF's loop uses: finished rows show `pad`; streamer.put; eos bookkeeping;
    stopping criteria on cat(prompt, tokens so far) (the reference's KeywordsStoppingCriteria looks at the tail of that
    tensor, llava/mm_utils.py:92-114). Returns a CPU int64 tensor [B, n], 1 <= n <= max_new_tokens."""
    Lt = prompt.shape[1]
    crit_buf = None
    if stopping_criteria:
        crit_buf = torch.empty(B, Lt + max_new_tokens, dtype=torch.long)
        crit_buf[:, :Lt] = prompt.to("cpu", torch.long)
    run_ahead = max(1, int(run_ahead))
    if not begun:  # generate() begins the stream itself (it confirms its input checks on token 0 before any output)
        engine.stream_begin(kv, logits, sampling)
    scheduled = 1                                   # tokens whose kernels have been queued (token 0 = begin)
    finished = [False] * B
    cols = []
    for t in range(max_new_tokens):
        # keep the device `run_ahead` tokens in front of the host (queued in blocks: one call per ~run_ahead/2 tokens)
        if scheduled < max_new_tokens and scheduled - t <= (run_ahead + 1) // 2:
            n = min(run_ahead - (scheduled - t) + 1, max_new_tokens - scheduled)
            if n > 0:
                engine.stream_enqueue(kv, n)
                scheduled += n
        toks = engine.stream_wait(kv, t, B)
        col = [pad if finished[b] else int(toks[b]) for b in range(B)]
        cols.append(col)
        if streamer is not None:
            streamer.put(torch.tensor(col, dtype=torch.long))
        for b in range(B):
            if col[b] in eos_ids:
                finished[b] = True
        stop = bool(eos_ids) and all(finished)
        if crit_buf is not None:
            crit_buf[:, Lt + t] = torch.tensor(col, dtype=torch.long)
            view = crit_buf[:, :Lt + t + 1]
            for crit in stopping_criteria:
                r = crit(view, None)
                stop = stop or (bool(r.all()) if torch.is_tensor(r) else bool(r))
        if stop:
            break
    return torch.tensor(cols, dtype=torch.long).t().contiguous()
