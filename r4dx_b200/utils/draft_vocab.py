"""Picks the token ids of a reduced-vocabulary draft head: the most frequent tokens of a text sample, plus ids that must
always be present (end-of-sequence, chat markers, tool-call tags).  The output is the JSON that ``convert --mtp
--draft-vocab-ids`` reads.

    python -m r4dx_b200.utils.draft_vocab --tokenizer-dir <dir> --text sample1.txt sample2.jsonl --size 32768 --out ids.json

The drafter only proposes tokens, and the verify pass scores the full vocabulary, so a token outside the list can still be
emitted: it just cannot be drafted, which costs acceptance, never correctness.  ``--coverage`` prints which share of the
sample's tokens the list covers (reference: the reduced-vocab draft head of src/convert/main.cpp:165-169 takes its ids from
a calibration run over tool-call transcripts).
"""
from __future__ import annotations

import argparse
import collections
import json
import sys
from typing import Iterable, List, Sequence


def pick_ids(token_streams: Iterable[Sequence[int]], size: int, always: Sequence[int] = (), vocab_size: int = 0) -> dict:
    counts: collections.Counter = collections.Counter()
    total = 0
    for toks in token_streams:
        counts.update(int(t) for t in toks)
        total += len(toks)
    keep: List[int] = []
    seen = set()
    for t in list(always) + [t for t, _ in sorted(counts.items(), key=lambda kv: (-kv[1], kv[0]))]:
        if t in seen or t < 0 or (vocab_size and t >= vocab_size):
            continue
        if len(keep) >= size:
            break
        keep.append(t)
        seen.add(t)
    covered = sum(c for t, c in counts.items() if t in seen)
    return {"ids": sorted(keep), "sample_tokens": total, "coverage": covered / max(1, total), "distinct_in_sample": len(counts)}


def _texts(paths: Sequence[str]) -> Iterable[str]:
    for p in paths:
        with open(p, encoding="utf-8") as f:
            if p.endswith(".jsonl"):
                for line in f:
                    if not line.strip():
                        continue
                    obj = json.loads(line)
                    if isinstance(obj, dict):
                        # request logs and chat transcripts: every string value at the top level or inside "messages"
                        for m in obj.get("messages", []):
                            if isinstance(m.get("content"), str):
                                yield m["content"]
                        for v in obj.values():
                            if isinstance(v, str):
                                yield v
                    elif isinstance(obj, str):
                        yield obj
            else:
                yield f.read()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("r4dxb-draft-vocab")
    ap.add_argument("--tokenizer-dir", default=None, help="tokenizer files (tokenizer.json ...); without it the byte-level test tokenizer")
    ap.add_argument("--vocab-size", type=int, default=4096)
    ap.add_argument("--text", nargs="+", required=True, help="plain text files, or .jsonl files of chat transcripts / request logs")
    ap.add_argument("--size", type=int, default=32768, help="ids to keep (the converter pads the count to a multiple of 128)")
    ap.add_argument("--always", default="", help="comma list of ids that are always kept (end-of-sequence, chat and tool-call markers)")
    ap.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    from ..runtime.tokenizer import load_tokenizer
    tk, _ = load_tokenizer(a.tokenizer_dir, a.vocab_size)
    always = [int(x) for x in a.always.split(",") if x]
    eos = getattr(tk, "eos_token_id", None)
    if isinstance(eos, int) and eos >= 0:
        always.append(eos)
    rep = pick_ids((tk.encode(t) for t in _texts(a.text)), a.size, always, getattr(tk, "vocab_size", 0) or a.vocab_size)
    json.dump({"ids": rep["ids"]}, open(a.out, "w"))
    print(json.dumps({k: v for k, v in rep.items() if k != "ids"} | {"kept": len(rep["ids"]), "out": a.out}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
