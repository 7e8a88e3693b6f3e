"""Layer-list decoders on the B200 engine: what every such model family shares on the Python side.

A checkpoint directory holds `config.json` (its `architecture` names the family, `layers` lists the layers) and
`model.safetensors`. A family module supplies a configuration class that turns config.json into the engine's model and
layer descriptions (include/b2llava.h, "layer-list decoders"); this module reads the tensors, hands everything to the engine
and offers `forward`, `generate` and the step-by-step replay. All arithmetic runs in libb2llava.so. Generation uses what every
model of the package uses: the cache pool, the device-resident decode loop with its host token ring, continuous batching.
"""
import json
import os
import struct
import threading

import torch

from ..._b2 import COMPUTE_BF16, COMPUTE_F32, LOGITS_ALL, LOGITS_LAST, SeqEngine, make_sampling
from ..._b2.generation import _KVPool, _stream_decode

_ST_DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path):
    """name -> CPU tensor. The file is an 8-byte little-endian header length, a JSON header (dtype, shape, data_offsets per
    tensor) and the raw data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        if meta["dtype"] not in _ST_DTYPES:
            raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
        lo, hi = meta["data_offsets"]
        t = torch.frombuffer(bytearray(data[lo:hi]), dtype=_ST_DTYPES[meta["dtype"]]) if hi > lo else torch.empty(0, dtype=_ST_DTYPES[meta["dtype"]])
        out[name] = t.reshape(meta["shape"])
    return out



class LayerListConfig:
    """Base of the families' configuration classes: `width`, `vocab`, `norm.eps`, `layers`; `layer_descs(shapes)` gives the
    engine's layer descriptions, `model_desc()` what the family adds to the engine's model description."""
    model_type = None

    def __init__(self, **cfg):
        if cfg.get("architecture", self.model_type) != self.model_type:
            raise ValueError(f"not a {self.model_type} configuration: architecture={cfg.get('architecture')!r}")
        self.raw = cfg
        self.width, self.vocab = int(cfg["width"]), int(cfg["vocab"])
        self.norm_eps = float(cfg["norm"]["eps"])
        self.layers = list(cfg["layers"])
        if not self.layers:
            raise ValueError(f"{self.model_type} configuration without layers")
        self.vocab_size, self.hidden_size = self.vocab, self.width
        self.eos_token_id = cfg.get("eos_token_id")

    @classmethod
    def from_pretrained(cls, path):
        with open(os.path.join(path, "config.json")) as f:
            return cls(**json.load(f))

    def model_desc(self):
        return {}

    def layer_descs(self, shapes):
        raise NotImplementedError


class LayerListForCausalLM:
    """Holds the checkpoint tensors (CPU) and builds the device engine on first use.

    dtype: torch.bfloat16 = bf16 matrix products with fp32 accumulation on bf16 weights (norms, scores, recurrences, the
    residual stream in fp32); torch.float32 = everything in true fp32."""
    config_class = LayerListConfig

    def __init__(self, config, tensors, device="cuda", dtype=torch.bfloat16, max_batch=1, max_seq=2048, max_rows=None):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"{config.model_type} runs in bfloat16 or float32")
        self.config, self.tensors, self.device, self.dtype = config, tensors, torch.device(device), dtype
        self._limits = {"max_batch": int(max_batch), "max_seq": int(max_seq), "max_rows": int(max_rows or max_seq)}
        self._engine = self._pool = self._batcher = None
        self._lock = threading.RLock()

    @classmethod
    def from_pretrained(cls, path, device="cuda", dtype=torch.bfloat16, torch_dtype=None, **limits):
        if not os.path.isdir(path):
            raise ValueError(f"{path!r} is not a local checkpoint directory")
        return cls(cls.config_class.from_pretrained(path), read_safetensors(os.path.join(path, "model.safetensors")), device=device,
                   dtype=torch_dtype or dtype, **limits)

    def eval(self):
        return self

    def engine_limits(self, max_batch=None, max_seq=None, max_rows=None):
        for k, v in (("max_batch", max_batch), ("max_seq", max_seq), ("max_rows", max_rows)):
            if v is not None and v != self._limits[k]:
                self._limits[k] = int(v)
                self.invalidate_engine()

    def invalidate_engine(self):
        with self._lock:
            if self._batcher is not None:
                self._batcher.close()
            if self._engine is not None:
                self._engine.close()
            self._engine = self._pool = self._batcher = None

    def _ensure_engine(self):
        if self._engine is not None:
            return self._engine
        with self._lock:
            if self._engine is not None:
                return self._engine
            c = self.config
            if self.device.type != "cuda":
                raise RuntimeError(f"{c.model_type} needs a CUDA (sm_100a) device; there is no CPU path")
            slots = max(self._limits["max_batch"], int(c.raw.get("b2_continuous_batching", 0) or 0))
            desc = dict(width=c.width, vocab=c.vocab, compute=COMPUTE_F32 if self.dtype == torch.float32 else COMPUTE_BF16,
                        norm_eps=c.norm_eps, max_batch=slots, max_rows=self._limits["max_rows"], **c.model_desc())
            eng = SeqEngine(desc, c.layer_descs({k: tuple(v.shape) for k, v in self.tensors.items()}), self.device)
            eng.max_seq = self._limits["max_seq"]
            for k, v in self.tensors.items():
                eng.set_weight(k, v)
            eng.finalize()
            self._pool = _KVPool(eng, slots, self._limits["max_seq"], int(c.raw.get("b2_max_concurrent_generations", 0) or 8))
            self._engine = eng
            return eng

    def _get_batcher(self, eng):
        slots = int(self.config.raw.get("b2_continuous_batching", 0) or 0)
        if slots < 2:
            return None
        with self._lock:
            if self._batcher is None:
                from ..._b2.batching import ContinuousBatcher
                self._batcher = ContinuousBatcher(eng, slots, self._limits["max_seq"])
            return self._batcher

    # ------------------------------------------------------------------ forward: logits of all positions
    @torch.no_grad()
    def forward(self, input_ids, output_hidden_states=False):
        """input_ids [B, S] (equal lengths) -> fp32 logits [B, S, vocab]; with output_hidden_states also the residual stream
        after every layer run [B, layer runs, S, width] (a looped layer counts every time)."""
        eng = self._ensure_engine()
        ids = input_ids if input_ids.dim() == 2 else input_ids.unsqueeze(0)
        kv = self._pool.acquire()
        try:
            logits, hidden = [], []
            for b in range(ids.shape[0]):
                row = ids[b].tolist()
                out = eng.append_tokens(kv, 0, row, list(range(len(row))), restart=True, residuals=output_hidden_states)
                if output_hidden_states:
                    logits.append(out[0]); hidden.append(out[1])
                else:
                    logits.append(out)
            torch.cuda.current_stream(self.device).synchronize()
            eng.check_async_error()
        finally:
            self._pool.release(kv)
        return (torch.stack(logits), torch.stack(hidden)) if output_hidden_states else torch.stack(logits)

    __call__ = forward

    # ------------------------------------------------------------------ generate
    @torch.no_grad()
    def generate(self, inputs=None, do_sample=False, temperature=1.0, top_p=None, top_k=None, max_new_tokens=20, streamer=None,
                 stopping_criteria=None, eos_token_id=None, pad_token_id=None, input_ids=None, num_beams=1, **kwargs):
        """Same protocol as the package's other generate(): prompt ids echoed in the result, streamer.put/end, stopping
        criteria called on the ids so far, eos stop, greedy or temperature / top-k / top-p selection on the device."""
        if kwargs:
            raise NotImplementedError(f"generate() got unsupported arguments {sorted(kwargs)}")
        if num_beams != 1:
            raise NotImplementedError("beam search")
        prompt = inputs if inputs is not None else input_ids
        if prompt is None:
            raise ValueError("generate() needs input ids")
        prompt = prompt if prompt.dim() == 2 else prompt.unsqueeze(0)
        B, Lt = prompt.shape
        if max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        eng = self._ensure_engine()
        if eos_token_id is None:
            eos_token_id = self.config.eos_token_id
        eos_ids = set(eos_token_id) if isinstance(eos_token_id, (list, tuple)) else ({eos_token_id} if eos_token_id is not None else set())
        pad = pad_token_id if pad_token_id is not None else (next(iter(eos_ids)) if eos_ids else 0)
        if (not do_sample) or (temperature is not None and temperature <= 1e-5):
            sampling = make_sampling()
        else:
            seed = int(torch.randint(0, 2**62, (1,), dtype=torch.int64).item())
            sampling = make_sampling(True, temperature, 1.0 if top_p is None else top_p, 50 if top_k is None else top_k, seed)
        if Lt + max_new_tokens > self._limits["max_seq"] or Lt > self._limits["max_rows"]:
            raise ValueError(f"{Lt} prompt + {max_new_tokens} new tokens exceed the engine limits {self._limits}; "
                             f"call model.engine_limits(...) before the first forward")
        batcher = self._get_batcher(eng) if B == 1 else None
        if batcher is not None:
            from ..._b2.batching import RequestStream
            req = batcher.submit(prompt.to("cpu", torch.int64), Lt, sampling, max_new_tokens)
            if streamer is not None:
                streamer.put(prompt.cpu())
            try:
                new = _stream_decode(RequestStream(req), None, None, sampling, 1, max_new_tokens, eos_ids, pad, prompt, streamer,
                                     stopping_criteria, begun=True)
            finally:
                req.cancel()
        else:
            if B > eng.desc.max_batch:
                raise ValueError(f"batch {B} exceeds the engine's {eng.desc.max_batch} slots")
            kv = self._pool.acquire()
            try:
                kv.reset()
                logits = eng.prefill(kv, prompt.to("cpu", torch.int64), None, LOGITS_LAST)
                eng.stream_begin(kv, logits, sampling)
                eng.stream_wait(kv, 0, B)
                eng.check_async_error()
                if streamer is not None:
                    streamer.put(prompt.cpu())
                new = _stream_decode(eng, kv, None, sampling, B, max_new_tokens, eos_ids, pad, prompt, streamer, stopping_criteria,
                                     run_ahead=int(self.config.raw.get("b2_run_ahead", 8)), begun=True)
            finally:
                self._pool.release(kv)
        if streamer is not None:
            streamer.end()
        return torch.cat([prompt, new.to(device=prompt.device, dtype=prompt.dtype)], dim=1)

    # ------------------------------------------------------------------ step-by-step replay (bin/trace_run)
    def trace_session(self):
        return TraceSession(self)


class TraceSession:
    """Given token ids in, logits out, one step at a time, on the engine's own paths: every request holds a slot of one
    cache; several tokens extend it through the prompt-portion call, one token of a running request through the decode
    step (the kernels generation uses); `end` gives the slot back."""

    def __init__(self, model):
        self.model, self.engine = model, model._ensure_engine()
        self.kv = model._pool.acquire()
        self.slots, self.free = {}, list(range(self.engine.desc.max_batch))[::-1]

    def feed(self, rid, tokens, want):
        eng = self.engine
        new = rid not in self.slots
        if new:
            if not self.free:
                raise RuntimeError(f"no free cache slot for request {rid!r} ({len(self.slots)} in flight)")
            self.slots[rid] = self.free.pop()
        slot = self.slots[rid]
        if len(tokens) == 1 and not new:
            logits = eng.decode_step(self.kv, torch.tensor(tokens, dtype=torch.int32), want_logits=True, slot0=slot)
            logits = logits if want else None
        else:
            logits = eng.append_tokens(self.kv, slot, tokens, want, restart=new)
        eng_err = eng.take_async_error() if want else 0
        if eng_err:
            raise ValueError("token id outside the vocabulary")
        return logits

    def sync(self):
        torch.cuda.current_stream(self.engine.device).synchronize()

    def end(self, rid):
        slot = self.slots.pop(rid)
        self.kv.free_slot(slot)
        self.free.append(slot)
