"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it
drives `EngineCore` (the model, step function, page pools and kernels that
generation uses). Steps arrive as JSON lines

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

and for a step that wants logits, `<out>/<step>.f32` holds them as little-endian
32-bit floats `[wanted, vocab]` in the order of the entries and of `want`.
After every step a line `done <step>` is printed and flushed.

The reference has no token-level replay; the nearest are its test harnesses that
feed one sequence in arbitrary pieces (src/provider/local/model/cpu.rs:3739-3877,
4072-4141).
"""
from __future__ import annotations

import json
import sys
from pathlib import Path


from .core import EngineCore
from .step import StepEntry

MAX_LIVE = 64


class Replayer:
    def __init__(self, core: EngineCore, out_dir):
        self.core = core
        self.out = Path(out_dir)
        self.out.mkdir(parents=True, exist_ok=True)
        self.live: dict = {}  # request id -> (SeqBlocks, slot)

    def run_step(self, record: dict) -> None:
        core = self.core
        entries = []
        for ent in record.get("entries", []):
            rid = ent["id"]
            tokens = [int(t) for t in ent["tokens"]]
            if not tokens:  # nothing to run for this request in this step
                if ent.get("want"):
                    raise ValueError(f"request `{rid}`, step {record['step']}: logits wanted of no tokens")
                continue
            if rid not in self.live:
                slot = core.slots.alloc()
                if slot is None:
                    raise RuntimeError(f"request `{rid}`: more than {core.max_sequences} live requests")
                core.cache.clear_slot(slot)
                self.live[rid] = (core.pools.new_seq(), slot)
            blocks, slot = self.live[rid]
            core.pools.reserve(blocks, blocks.length + len(tokens))
            entries.append(StepEntry(blocks, slot, tokens, [int(w) for w in ent.get("want", [])]))
        if entries:
            logits = core.stepper.step(entries)
            core.rt.check_device_errors()
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                arr.tofile(self.out / f"{record['step']}.f32")
        for rid in record.get("end", []):
            if rid in self.live:
                blocks, slot = self.live.pop(rid)
                core.pools.release(blocks)
                core.slots.release(slot)

    def run(self, lines, echo=sys.stdout) -> None:
        for line in lines:
            line = line.strip()
            if not line:
                continue
            record = json.loads(line)
            self.run_step(record)
            print(f"done {record['step']}", file=echo, flush=True)


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--block-size", type=int, default=16, help="positions per page")
    args = ap.parse_args(argv)
    # --max-tokens counts every live request's tokens rounded up to 64; with larger pages each of those 64 may be a
    # request of its own that needs a whole page
    kv_tokens = -(-args.max_tokens // 64) * max(64, args.block_size)
    core = EngineCore.from_folder(args.model, dtype=args.dtype, kv_tokens=kv_tokens, max_sequences=MAX_LIVE,
                                  block_size=args.block_size, window_pools="full")
    Replayer(core, args.out).run(sys.stdin)
    return 0
