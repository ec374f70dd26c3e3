"""N-gram speculation simulator: replays finished generations and reports what a prompt-lookup drafter would have saved.

    python -m r4dx_b200.utils.ngram_sim --log requests.jsonl [--k 4] [--min-n 2] [--max-n 4]

Each line of the log is a JSON object with ``prompt_ids`` and ``completion_ids`` (what the server's request log writes when
it is started with token logging; ``token_ids`` is accepted too).  Prints one JSON line per request and a total.
(reference: tools/ngram, the n-gram speculation simulator.)"""
from __future__ import annotations

import argparse
import json
import sys

from ..models.ngram import simulate


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("r4dxb-ngram-sim")
    ap.add_argument("--log", required=True)
    ap.add_argument("--k", type=int, default=4)
    ap.add_argument("--min-n", type=int, default=2)
    ap.add_argument("--max-n", type=int, default=4)
    a = ap.parse_args(argv)
    tot_out, tot_calls = 0, 0
    for line in open(a.log):
        line = line.strip()
        if not line:
            continue
        d = json.loads(line)
        prompt, out = list(d.get("prompt_ids", [])), list(d.get("completion_ids", d.get("token_ids", [])))
        if not out:
            continue
        s = simulate(prompt + out, len(prompt), a.k, a.min_n, a.max_n)
        print(json.dumps(s))
        tot_out += s["output_tokens"]
        tot_calls += s["target_calls"]
    print(json.dumps({"total_output_tokens": tot_out, "total_target_calls": tot_calls,
                      "tokens_per_call": tot_out / max(1, tot_calls)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
