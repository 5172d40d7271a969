"""The library entry in the reference's manner: `LocalModel.load(config)` then `generate(...)`
(src/provider/local/mod.rs:2423,3213,3276). Token ids in, token ids out: chat templates and tokenizers are
outside this engine."""
from __future__ import annotations

import json
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Optional, Sequence

import torch

from ..config.engine_config import LocalModelConfig, SamplingConfig
from ..config.model_config import read_config_json
from ..config.registry import build_spec
from ..kernels import ops
from ..weights.loader import FolderSource
from .core import EngineCore
from .graphs import MAX_HISTORY, DecodeGraphs
from .scheduler import Plan, Request, Scheduler, SchedulerConfig, Sequence_
from .step import StepEntry
from .stop import StopMatcher
from .text import TextCodec, TextStream


@dataclass
class Usage:
    prompt_tokens: int
    completion_tokens: int


@dataclass
class GenerationReport:
    """src/provider/local/mod.rs:3155-3168: exact token counts, why it stopped, how long it queued."""

    usage: Usage
    finish_reason: str  # "stop" | "length" | "error"
    queue_secs: float
    error: Optional[str] = None
    preemptions: int = 0


@dataclass
class LocalGeneration:
    tokens: list
    report: GenerationReport
    text: Optional[str] = None  # with a tokenizer attached: the reply, cut before a stop string


class GpuBackend:
    """Runs the scheduler's plans on the device: one step, then one sampled token per wanted row."""

    def __init__(self, core: EngineCore):
        self.core = core
        dev = core.rt.device
        n = core.max_sequences
        self.rng = torch.zeros(n, dtype=torch.int64, device=dev)
        self.temperature = torch.zeros(n, dtype=torch.float32, device=dev)
        self.top_k = torch.zeros(n, dtype=torch.int32, device=dev)
        self.top_p = torch.ones(n, dtype=torch.float32, device=dev)
        self._scratch = None
        self.suppress = None  # int32 ids whose logits are set to -inf before sampling
        self._needs_scratch = [False] * n
        self.sample_split = ops.SampleSplit(max(n, 64), dev)  # greedy rows of a large vocabulary: several CTAs a row
        self.vocab = core.spec.vocab_size
        self.use_graphs = core.model.graph_safe()
        self.graphs = DecodeGraphs(core, self)
        self.graph_steps = 0
        self.eager_steps = 0
        self.last_graph = None  # the captured step that ran last
        self.h2d_bytes = 0  # bytes of step inputs copied to the device (besides the step function's own uploads)
        self.d2h_bytes = 0  # bytes of sampled tokens (and the error word) read back

    def start(self, seq: Sequence_) -> None:
        """A request takes its slot: clear its state, set its sampling constants and its generator."""
        r, s = seq.request, seq.slot
        self.core.cache.clear_slot(s)
        state = seq.rng_state()
        self.rng[s] = state - (1 << 64) if state >= (1 << 63) else state
        self.temperature[s] = float(r.temperature)
        self.top_k[s] = int(r.top_k)
        self.top_p[s] = float(r.top_p)
        ranked = 0 < r.top_k < self.vocab
        self._needs_scratch[s] = r.temperature > 0 and ((ranked and r.top_k > 1024) or (not ranked and r.top_p < 1.0))

    # ------------------------------------------------------------ decode through a captured graph
    def _run_decode_graph(self, plans: Sequence[Plan]) -> list:
        seqs = [p.seq for p in plans]
        n = len(seqs)
        starts = [p.start if p.start >= 0 else p.seq.blocks.length for p in plans]
        max_len = max(starts) + 1
        g = self.graphs.get(n, max_len, any(self._needs_scratch[s.slot] for s in seqs))
        stepper = self.core.stepper
        handles, slots, tokens = [s.blocks.handle for s in seqs], [s.slot for s in seqs], [p.tokens[0] for p in plans]
        advance = stepper.single_token_step(handles, slots, tokens)  # an eager step's refusals, the page tables
        g.load_rows(tokens, starts, slots)
        g.replay()
        self.last_graph = g
        self.h2d_bytes += 4 * g.meta.numel()
        self.d2h_bytes += 4 * g.sampled.numel()
        out = g.sampled.tolist()  # the one synchronisation of a step; its last word is the device error word
        if out[g.bucket]:
            self.core.rt.raise_device_error(out[g.bucket])  # before anything is applied: the step is lost
        tokens = out[:n]
        advance()
        self.core.stepper.steps += 1
        self.graph_steps += 1
        return tokens

    def burst(self, seqs, tokens, n_steps: int, check: bool = True):
        """`n_steps` decode steps back to back on the device, each feeding its sampled tokens to the next; the
        host only reserves pages ahead and reads the tokens at the end. Returns a [n_steps, requests] tensor.
        With `check` the device error word is read after the last step (one synchronisation) and a recorded fault
        raises before any request advances."""
        core = self.core
        n = len(seqs)
        if n_steps > MAX_HISTORY:
            raise ValueError(f"a burst holds at most {MAX_HISTORY} steps")
        starts = [s.blocks.length for s in seqs]
        for s, start in zip(seqs, starts):
            core.pools.reserve(s.blocks, start + n_steps)
        max_len = max(starts) + n_steps
        g = self.graphs.get(n, max_len, any(self._needs_scratch[s.slot] for s in seqs))
        stepper = core.stepper
        handles, slots = [s.blocks.handle for s in seqs], [s.slot for s in seqs]
        stepper.check_single_tokens(handles, slots, tokens)
        stepper.upload_table_updates(handles, slots)
        g.load_rows(tokens, starts, slots)
        g.counter.zero_()
        for _ in range(n_steps):
            g.replay()
        if check:
            code = int(g.sampled[g.bucket].item())
            if code:
                self.core.rt.raise_device_error(code)
        stepper.advance(handles, [n_steps] * n)
        self.graph_steps += n_steps
        return g.history[:n_steps, :n]

    def run(self, plans: Sequence[Plan]) -> list:
        if self.use_graphs and all(len(p.tokens) == 1 and p.want_last for p in plans):
            return self._run_decode_graph(plans)
        self.eager_steps += 1
        entries = [StepEntry(p.seq.blocks, p.seq.slot, p.tokens, [len(p.tokens) - 1] if p.want_last else [])
                   for p in plans]
        logits = self.core.stepper.step(entries)
        if logits is None:
            return []
        rows = [p.seq.slot for p in plans if p.want_last]
        slot_of_row = torch.tensor(rows, dtype=torch.int32).to(self.core.rt.device, non_blocking=True)
        out = torch.empty(len(rows), dtype=torch.int32, device=self.core.rt.device)
        scratch = None
        if any(self._needs_scratch[s] for s in rows):
            words = ops.sample_scratch_words(self.vocab)
            if self._scratch is None or self._scratch.shape[0] < len(rows):
                self._scratch = torch.empty(max(len(rows), 4), words, dtype=torch.int64, device=self.core.rt.device)
            scratch = self._scratch
        if self.suppress is not None:
            ops.suppress_tokens(logits, self.suppress)
        ops.sample(logits, self.temperature, self.top_k, self.top_p, self.rng, slot_of_row, out, scratch,
                   self.sample_split)
        tokens = out.tolist()  # the one synchronisation of a step
        self.h2d_bytes += 4 * len(rows)
        self.d2h_bytes += 4 * len(rows) + 4
        self.core.rt.check_device_errors()
        return tokens


def _file_sampling(model_dir: Optional[Path]) -> dict:
    """generation_config.json of the checkpoint: its temperature, top_k, top_p (src/provider/local/sampling.rs:8-32)."""
    if model_dir is None:
        return {}
    f = Path(model_dir) / "generation_config.json"
    if not f.is_file():
        return {}
    try:
        g = json.loads(f.read_text())
    except ValueError:
        return {}
    return {k: g[k] for k in ("temperature", "top_k", "top_p", "suppress_tokens") if g.get(k) is not None}


class LocalModel:
    """A loaded model with its scheduler. One process, one GPU, one engine."""

    def __init__(self, core: EngineCore, config: LocalModelConfig, sizes: dict, model_dir: Optional[Path]):
        self.core = core
        self.config = config
        self.sizes = sizes
        self.backend = GpuBackend(core)
        if self.backend.use_graphs:
            self.backend.graphs.prime(config.batching.max_sequences)
        self.scheduler = Scheduler(core.pools, core.slots, self.backend, SchedulerConfig(
            max_sequences=config.batching.max_sequences, max_step_tokens=sizes["max_step_tokens"],
            prefill_chunk=sizes["prefill_chunk"], context_length=sizes["context_length"],
            eos_token_ids=tuple(core.spec.eos_token_ids), prefix_cache=bool(config.batching.prefix_cache)))
        self._file_sampling = _file_sampling(model_dir)
        suppressed = config.sampling.suppress_tokens
        if suppressed is None:
            suppressed = self._file_sampling.get("suppress_tokens")
        if suppressed:
            self.backend.suppress = torch.tensor([int(t) for t in suppressed], dtype=torch.int32,
                                                 device=core.rt.device)
        self.text = TextCodec.find(model_dir)  # None: token ids only
        self.load_seconds = 0.0

    # ------------------------------------------------------------ loading
    @classmethod
    def load(cls, config: LocalModelConfig) -> "LocalModel":
        t0 = time.perf_counter()
        config.validate()
        if config.source is not None:
            model_dir = Path(config.source)
            cfg_json = read_config_json(model_dir)
        else:
            model_dir, cfg_json = None, config.model_config
        spec = build_spec(cfg_json)
        sizes = config.resolve(spec.max_positions)
        kw = dict(dtype=config.dtype, device=config.device, context_length=sizes["context_length"],
                  kv_tokens=sizes["kv_tokens"], max_sequences=config.batching.max_sequences,
                  block_size=config.kv_block_size, max_step_tokens=sizes["max_step_tokens"])
        if model_dir is not None:
            core = EngineCore(spec, FolderSource(model_dir), **kw)
        else:
            core = EngineCore(spec, None, random_seed=config.random_weights.seed,
                              random_std=config.random_weights.std, **kw)
        model = cls(core, config, sizes, model_dir)
        model.load_seconds = time.perf_counter() - t0
        return model

    # ------------------------------------------------------------ requests
    def _request(self, prompt, max_tokens, temperature, top_k, top_p, seed, stop_token_ids) -> Request:
        """request > config.sampling > the checkpoint's generation_config.json > 1.0 / 64 / 0.95
        (src/provider/local/sampling.rs:1-19,93-111)."""
        s, f = self.config.sampling, self._file_sampling

        def pick(req, cfg, key, default):
            if req is not None:
                return req
            if cfg is not None:
                return cfg
            return f.get(key, default)

        return Request(
            prompt=list(prompt), max_tokens=max_tokens,
            temperature=float(pick(temperature, s.temperature, "temperature", SamplingConfig.DEFAULT_TEMPERATURE)),
            top_k=int(pick(top_k, s.top_k, "top_k", SamplingConfig.DEFAULT_TOP_K)),
            top_p=float(pick(top_p, s.top_p, "top_p", SamplingConfig.DEFAULT_TOP_P)),
            seed=seed if seed is not None else s.seed, stop_token_ids=tuple(stop_token_ids or ()))

    def tokenize(self, text: str) -> list:
        """Token ids of `text` (src/provider/local/mod.rs:3213); needs the folder's tokenizer."""
        if self.text is None:
            raise ValueError("this model folder has no tokenizer.json: prompts are lists of token ids")
        return self.text.encode(text)

    def generate(self, prompts, max_tokens: Optional[int] = None, temperature: Optional[float] = None,
                 top_k: Optional[int] = None, top_p: Optional[float] = None, seed: Optional[int] = None,
                 stop_token_ids: Iterable[int] = (), on_token=None, stop: Iterable[str] = (), on_text=None):
        """Generate for one prompt (a list of token ids) or several (a list of lists); returns one
        `LocalGeneration` or a list of them, in the order given. All prompts run together under continuous
        batching. With a tokenizer in the model folder a prompt may be a string, the results carry their text,
        `on_text(sequence, fragment)` streams it, and `stop` strings cut the reply before their first occurrence
        (finish reason "stop"; src/provider/local/engine/stop.rs, scheduler.rs:92-136)."""
        single = isinstance(prompts, str) or (len(prompts) > 0 and not isinstance(prompts[0], (list, tuple, str)))
        batch = [prompts] if single else list(prompts)
        batch = [self.tokenize(p) if isinstance(p, str) else p for p in batch]
        stop = [s for s in (stop or ()) if s]
        if stop and self.text is None:
            raise ValueError("stop strings need the model folder's tokenizer.json; use stop_token_ids")
        seqs = [self.scheduler.submit(self._request(p, max_tokens, temperature, top_k, top_p, seed, stop_token_ids))
                for p in batch]
        if self.text is None:
            self.scheduler.run_until_done(on_token)
            texts = {}
        else:
            texts = self._run_with_text(seqs, stop, on_token, on_text)
        out = [LocalGeneration(list(s.completion), GenerationReport(
            Usage(s.prompt_tokens, len(s.completion)), s.finish_reason or "error",
            max(0.0, s.started_at - s.queued_at), s.error, s.preemptions), texts.get(id(s))) for s in seqs]
        for s in seqs:
            if s in self.scheduler.finished:
                self.scheduler.finished.remove(s)
        return out[0] if single else out

    def _run_with_text(self, seqs, stop, on_token, on_text) -> dict:
        """Runs the scheduler until these requests are done, turning their tokens into text as they come. A
        request whose text completes a stop string is cancelled after the turn that sampled it (the scheduler
        reports tokens from inside its own bookkeeping, so nothing is cancelled from the callback) and ends as
        "stop" with the text before the stop string."""
        streams = {id(s): (TextStream(self.text), StopMatcher(stop)) for s in seqs}
        texts = {id(s): "" for s in seqs}
        stopped, stopped_ids = [], set()

        def emit(seq, fragment):
            if fragment:
                texts[id(seq)] += fragment
                if on_text:
                    on_text(seq, fragment)

        def token(seq, tok):
            if on_token:
                on_token(seq, tok)
            pair = streams.get(id(seq))
            if pair is None or id(seq) in stopped_ids:
                return
            fragment, done = pair[1].push(pair[0].push(seq.completion))
            emit(seq, fragment)
            if done:
                stopped.append(seq)
                stopped_ids.add(id(seq))

        sched = self.scheduler
        sched._on_token = token
        while sched.has_work():
            progressed = sched.turn()
            for seq in stopped:
                if not seq.done:
                    sched.cancel(seq)
                    seq.finish_reason = "stop"
            if progressed == 0 and sched.has_work():
                raise RuntimeError("the scheduler made no progress: the page pool is too small for the queue's head")
        for s in seqs:
            if id(s) not in stopped_ids:
                emit(s, streams[id(s)][1].flush())
        return texts

    def generate_tokens(self, prompt, **kw):
        """Stream one request's tokens as they are sampled (src/provider/local/mod.rs:3276)."""
        seq = self.scheduler.submit(self._request(
            prompt, kw.get("max_tokens"), kw.get("temperature"), kw.get("top_k"), kw.get("top_p"), kw.get("seed"),
            kw.get("stop_token_ids", ())))
        sent = 0
        while True:
            while sent < len(seq.completion):
                yield seq.completion[sent]
                sent += 1
            if seq.done:
                break
            self.scheduler.turn()
        if seq in self.scheduler.finished:
            self.scheduler.finished.remove(seq)

    # ------------------------------------------------------------ facts
    def serving_stats(self):
        return self.scheduler.stats

    def kv_cache_bytes(self) -> int:
        return self.core.cache.bytes()

    def context_length(self) -> int:
        return self.sizes["context_length"]


def generate(model, prompts, **kw):
    """`generate(model_dir | LocalModelConfig | LocalModel, prompts, max_tokens=..., temperature=..., top_k=...,
    top_p=..., seed=..., stop_token_ids=...)`: load if needed, then generate."""
    if isinstance(model, (str, Path)):
        model = LocalModel.load(LocalModelConfig(source=str(model)))
    elif isinstance(model, LocalModelConfig):
        model = LocalModel.load(model)
    return model.generate(prompts, **kw)
