"""Builds replay traces (the four work splits) and compares replayed logits with the plain implementation."""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

import plain_llama

ROOT = Path(__file__).resolve().parent.parent


def round64(n: int) -> int:
    return -(-n // 64) * 64


# ---------------------------------------------------------------- traces
def trace_whole(requests: dict) -> list:
    """Each request alone and whole: one step with every position wanted."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def trace_tail_one_by_one(requests: dict, tail: int = 32) -> list:
    """Most of a request in one step, the last `tail` tokens one by one."""
    steps, n = [], 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": [head - 1]}], "end": []})
        n += 1
        for i in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: dict, sizes=(5, 2, 17, 3, 2, 32, 7, 2, 64, 11)) -> list:
    """Portions of changing size, down to two tokens; the last place of each portion is wanted."""
    steps, n = [], 0
    for rid, toks in requests.items():
        pos, k = 0, 0
        while pos < len(toks):
            size = min(sizes[k % len(sizes)], len(toks) - pos)
            k += 1
            last = pos + size == len(toks)
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[pos:pos + size],
                                                   "want": [0, size - 1] if size > 1 else [0]}],
                          "end": [rid] if last else []})
            pos += size
            n += 1
    return steps


def trace_mixed(requests: dict, max_live: int = 4, seed: int = 0, prefill_sizes=(9, 2, 30, 5, 16)) -> list:
    """Up to `max_live` live requests; portions of some beside single tokens of others; requests sit out at
    random."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live = {}  # rid -> [tokens, pos, decode_from]
    steps, n = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0, max(1, len(toks) - int(rng.integers(4, 20)))]
        entries, ended = [], []
        for rid in list(live):
            toks, pos, decode_from = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue  # sits this step out
            if pos < decode_from:
                size = min(int(prefill_sizes[int(rng.integers(len(prefill_sizes)))]), decode_from - pos)
                if decode_from - pos - size == 1:
                    size += 1  # never leave a one-token portion of the prompt
            else:
                size = 1
            entries.append({"id": rid, "tokens": toks[pos:pos + size], "want": [size - 1]})
            live[rid][1] = pos + size
            if pos + size == len(toks):
                ended.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": n, "entries": entries, "end": ended})
            n += 1
    return steps


def peak_tokens(steps: list) -> int:
    live, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            live[e["id"]] = live.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(round64(v) for v in live.values()))
        for rid in s["end"]:
            live.pop(rid, None)
    return peak


# ---------------------------------------------------------------- running
def run_in_process(model_dir, dtype: str, steps: list, max_tokens: int, block_size: int = 16) -> dict:
    """Replay through the framework's Replayer in this process; returns step -> logits [wanted, vocab]."""
    from cuca_b200.engine.core import EngineCore
    from cuca_b200.engine.replay import MAX_LIVE, Replayer

    out = tempfile.mkdtemp(prefix="replay_out_")
    core = EngineCore.from_folder(model_dir, dtype=dtype, kv_tokens=round64(max_tokens), max_sequences=MAX_LIVE,
                                  block_size=block_size, window_pools="full")
    rp = Replayer(core, out)
    with open(os.devnull, "w") as sink:
        rp.run([json.dumps(s) for s in steps], echo=sink)
    core.pools.check()
    assert core.pools.stats()["live_requests"] == 0
    assert all(p.free == p.n_blocks for p in core.pools.pools), "pages were lost"
    return read_outputs(out, steps, core.spec.vocab_size)


def run_subprocess(model_dir, dtype: str, steps: list, max_tokens: int, env=None) -> dict:
    """Replay through bin/trace_run as a user would."""
    out = tempfile.mkdtemp(prefix="replay_out_")
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", out, "--max-tokens", str(max_tokens)]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run(cmd, input=text, capture_output=True, text=True, env=env, timeout=900)
    assert r.returncode == 0, f"trace_run failed:\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps]
    vocab = json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]
    return read_outputs(out, steps, vocab)


def read_outputs(out_dir, steps: list, vocab: int) -> dict:
    got = {}
    for s in steps:
        wanted = sum(len(e.get("want", [])) for e in s["entries"])
        f = Path(out_dir) / f"{s['step']}.f32"
        if wanted == 0:
            assert not f.exists()
            continue
        arr = np.fromfile(f, dtype="<f4")
        assert arr.size == wanted * vocab, f"step {s['step']}: {arr.size} floats for {wanted} places"
        got[s["step"]] = arr.reshape(wanted, vocab)
    return got


# ---------------------------------------------------------------- comparing
class Oracle:
    """Plain whole-sequence logits of every request (cached per request)."""

    def __init__(self, model_dir):
        self.cfg, self.weights = plain_llama.load_model_dir(model_dir)
        self._cache = {}

    def logits(self, rid: str, tokens: list) -> np.ndarray:
        if rid not in self._cache:
            self._cache[rid] = plain_llama.forward(self.cfg, self.weights, tokens).numpy()
        return self._cache[rid]


def compare(steps: list, got: dict, requests: dict, oracle: Oracle, rel_tol: float) -> float:
    """Every wanted place against the oracle: max |diff| <= rel_tol * max |oracle logit of that row|.
    Reports the first wrong token with its place. Returns the worst ratio seen."""
    pos = {rid: 0 for rid in requests}
    worst = 0.0
    for s in steps:
        row = 0
        for e in s["entries"]:
            rid, n = e["id"], len(e["tokens"])
            ref = oracle.logits(rid, requests[rid])
            for w in e.get("want", []):
                p = pos[rid] + w
                r, g = ref[p], got[s["step"]][row]
                assert np.isfinite(g).all(), f"step {s['step']} request {rid} position {p}: non-finite logits"
                err = float(np.abs(g - r).max()) / float(np.abs(r).max())
                worst = max(worst, err)
                assert err <= rel_tol, (
                    f"first wrong token: step {s['step']}, request {rid}, position {p} (portion starts at "
                    f"{pos[rid]}, place {w} of {n}): relative error {err:.3e} > {rel_tol:.1e}")
                row += 1
            pos[rid] += n
    return worst
