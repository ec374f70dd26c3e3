"""r4dxb-cli: one-shot or interactive generation (reference: src/cli/main.cpp:128,557,969)."""
from __future__ import annotations

import sys
import time

from .args import cli_parser


def image_prompt(tm, tk, tpl, messages, files, think: bool):
    """Renders a prompt whose last user message starts with the given image files: every image becomes as many placeholder
    tokens as the vision tower yields rows for it, and those rows override the placeholders' embeddings
    (reference: src/cli/main.cpp:128, the --image path).  Returns (token ids, (positions, rows))."""
    import numpy as np
    import torch
    from PIL import Image
    from ..models.vision import VisionConfig, VisionTower, init_vision_weights
    from ..runtime import image_prompt as IP
    imgs = [torch.from_numpy(np.asarray(Image.open(f).convert("RGB"), dtype=np.uint8).copy()) for f in files]
    vw = {k[len("vision."):]: v for k, v in getattr(tm.m, "w", {}).items() if isinstance(k, str) and k.startswith("vision.")}
    vcfg = VisionConfig.from_weights(vw) if vw else None
    if not vw:                                   # synthetic models get a synthetic tower
        vcfg = VisionConfig(depth=2, hidden_size=144, num_heads=2, intermediate_size=256, patch_size=8,
                            out_hidden_size=tm.config.hidden_size, num_position_embeddings=64, max_pixels=256 * 256)
        vw = init_vision_weights(vcfg, 0)
    tower = VisionTower(vcfg, vw, device=str(tm.m.device))
    image_id = getattr(tk, "image_pad_id", tm.config.vocab_size - 1)
    msgs = [dict(m) for m in messages]
    msgs[-1]["content"] = "".join(IP.MARK % i for i in range(len(imgs))) + msgs[-1]["content"]
    text = tpl.render(msgs, add_generation_prompt=True, enable_thinking=think)
    spans = [(IP.MARK % i, image_id, IP.image_token_count(im, vcfg)) for i, im in enumerate(imgs)]
    ids = IP.assemble_media_prompt(text, spans, tk.encode)
    rows = tower.encode_images(imgs)
    where = torch.tensor([i for i, t in enumerate(ids) if t == image_id], dtype=torch.long)
    if where.numel() != rows.shape[0]:
        raise ValueError(f"{where.numel()} image placeholder tokens for {rows.shape[0]} image rows")
    return ids, (where, rows)


def run_turn(tm, tk, prompt_ids, args, rng, out=sys.stdout, embed_overrides=None):
    """Prefill + decode one answer; returns (token ids, stats dict)."""
    from ..runtime.sampler import SampleParams
    from ..runtime.tokenizer import StreamDecoder
    params = SampleParams(args.temperature, args.top_k, args.top_p, args.min_p, args.seed, args.repetition_penalty)
    t0 = time.perf_counter()
    tok = tm.prefill(prompt_ids, embed_overrides=embed_overrides) if embed_overrides is not None else tm.prefill(prompt_ids)
    if not params.greedy:
        tok = tm.sample_from_last(params, rng, prompt_ids)
    t1 = time.perf_counter()
    eos = set(getattr(tk, "eos_ids", []))
    dec = StreamDecoder(tk)
    ids, rounds = [], 0
    pending = [tok]
    while pending and len(ids) < args.max_tokens:
        tok = pending.pop(0)
        if tok in eos:
            break
        ids.append(tok)
        out.write(dec.feed(tok)); out.flush()
        if not pending:
            rounds += 1
            spec_k = args.mtp or getattr(args, "ngram", 0) or (args.dflash_k if getattr(args, "dflash", None) else 0)
            if spec_k > 0 and params.greedy:
                pending = tm.decode_step_spec_greedy(tok, spec_k)
            elif spec_k > 0:
                pending = tm.decode_step_spec_sampled(tok, spec_k, params, rng, list(prompt_ids) + ids[:-1])
            elif params.greedy:
                pending = [tm.decode_step_greedy(tok)]
            else:
                pending = [tm.decode_step_sampled(tok, params, rng, list(prompt_ids) + ids)]
    out.write(dec.flush() + "\n")
    t2 = time.perf_counter()
    stats = {"prompt_tokens": len(prompt_ids), "prefill_tok_s": len(prompt_ids) / max(t1 - t0, 1e-9),
             "ttft_s": t1 - t0, "decode_tokens": len(ids), "decode_tok_s": max(len(ids) - 1, 0) / max(t2 - t1, 1e-9),
             "tokens_per_round": len(ids) / max(rounds, 1)}
    return ids, stats


def main(argv=None) -> int:
    args = cli_parser().parse_args(argv)
    from ..runtime.sampler import Rng
    from .loader import load_text_model
    tm, tk, tpl = load_text_model(args)
    if tm.tp_world() > 1 and getattr(tm, "rank", 0) != 0:
        tm.follow()                      # follower rank: replay the leader's commands, print nothing
        return 0
    import atexit
    if hasattr(tm, "shutdown"):
        atexit.register(tm.shutdown)     # releases the follower ranks when the leader is done
    rng = Rng(args.seed)
    if args.profile or args.profile_prefill:
        from ..utils.profiler import profile_decode_step, profile_prefill
        ids = tk.encode(args.prompt or "hello")
        print(profile_prefill(tm.m, ids) if args.profile_prefill else profile_decode_step(tm.m, ids))
        return 0

    def build(messages):
        text = tpl.render(messages, add_generation_prompt=True, enable_thinking=(args.think == "on"))
        return tk.encode(text)

    messages = []
    if args.system:
        messages.append({"role": "system", "content": args.system})
    if args.chat:
        while True:
            try:
                line = input("> ")
            except EOFError:
                break
            if not line.strip():
                continue
            messages.append({"role": "user", "content": line})
            tm.reset()
            ids, stats = run_turn(tm, tk, build(messages), args, rng)
            messages.append({"role": "assistant", "content": tk.decode(ids)})
            if args.stats:
                print(f"[stats] {stats}", file=sys.stderr)
        return 0
    prompt = args.prompt if args.prompt is not None else (open(args.prompt_file).read() if args.prompt_file else "Hello")
    messages.append({"role": "user", "content": prompt})
    overrides = None
    if args.image:
        if args.vision != "on":
            print("--image needs --vision on", file=sys.stderr)
            return 2
        pids, overrides = image_prompt(tm, tk, tpl, messages, args.image, args.think == "on")
    else:
        pids = build(messages)
    if args.dump_token_ids:
        print(pids, file=sys.stderr)
    ids, stats = run_turn(tm, tk, pids, args, rng, embed_overrides=overrides)
    if args.stats:
        print(f"[stats] prefill {stats['prefill_tok_s']:.1f} tok/s (TTFT {stats['ttft_s'] * 1e3:.1f} ms), decode "
              f"{stats['decode_tok_s']:.1f} tok/s, {stats['tokens_per_round']:.2f} tokens/round, tp={tm.tp_world()}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
