"""r4dxb-server entry point (reference: src/server/main.cpp)."""
from __future__ import annotations

import sys

from .args import server_parser


def main(argv=None) -> int:
    args = server_parser().parse_args(argv)
    from ..server.engine import Engine
    from ..server.http_server import ApiServer
    from ..server.request_log import RequestLog
    from .loader import load_text_model
    tm, tk, tpl = load_text_model(args)
    if tm.tp_world() > 1 and getattr(tm, "rank", 0) != 0:
        # follower rank of a tensor-parallel group: no HTTP port, no engine - replay the leader's commands until it stops
        tm.follow()
        return 0
    if args.batch > 1 and tm.tp_world() > 1:
        raise SystemExit("--batch with --tp is not supported: the slot scheduler runs on one rank")
    if args.batch > 1:
        # N sequence slots over the same weights; the single-sequence model object only lends its weights
        from ..models.batch import BatchModel
        from ..server.batch_executor import BatchEngine
        m = tm.m
        bm = BatchModel(m.cfg, m.w, slots=args.batch, slot_ctx=args.batch_ctx, device=str(m.device), comm=m.comm)
        eng = BatchEngine(bm, tk, max_queue=max(args.max_queue, 2 * args.batch),
                          request_log=RequestLog(args.request_log, args.request_log_tokens))
    else:
        eng = Engine(tm, tk, max_queue=args.max_queue, prompt_checkpoint=(args.prompt_checkpoint == "on"),
                     request_log=RequestLog(args.request_log, args.request_log_tokens))
    vision, vcfg, image_id = None, None, -1
    if args.vision == "on" and args.batch <= 1:
        # the tower's weights ride in the container under "vision."; synthetic models get a synthetic tower
        from ..models.vision import VisionConfig, VisionTower, init_vision_weights
        vw = {k[len("vision."):]: v for k, v in getattr(tm.m, "w", {}).items() if isinstance(k, str) and k.startswith("vision.")}
        if tm.config.arch == "gemma":
            # encoder-free embedder of this family: the front object sizes the images and marks their rows as blocks
            from ..models.gemma_vision import GemmaVisionFront, random_embedder_weights
            vision = (GemmaVisionFront.from_container_tensors(vw, str(tm.m.device)) if vw
                      else GemmaVisionFront(random_embedder_weights(tm.config.hidden_size), str(tm.m.device)))
            if getattr(args, "image_soft_tokens", 0):
                from ..models.gemma_vision import SOFT_TOKEN_BUDGETS
                if args.image_soft_tokens not in SOFT_TOKEN_BUDGETS:
                    raise SystemExit(f"--image-soft-tokens must be one of {SOFT_TOKEN_BUDGETS}")
                vision.max_soft_tokens = args.image_soft_tokens
            vcfg, vw = vision, None
        else:
            vcfg = VisionConfig.from_weights(vw) if vw else None
        if vision is None and not vw:
            vcfg = VisionConfig(depth=2, hidden_size=144, num_heads=2, intermediate_size=256, patch_size=8,
                                out_hidden_size=tm.config.hidden_size, num_position_embeddings=64, max_pixels=256 * 256)
            vw = init_vision_weights(vcfg, 0)
        if vision is None:
            if getattr(args, "image_max_pixels", 0):
                vcfg.max_pixels = max(vcfg.min_pixels, min(vcfg.max_pixels, args.image_max_pixels))
            vision = VisionTower(vcfg, vw, device=str(tm.m.device))
        image_id = getattr(tk, "image_pad_id", tm.config.vocab_size - 1)
        eng.vision = vision
    from ..server.parsers import select_dialect
    eng.dialect = getattr(args, "dialect", "auto")
    warn = select_dialect(eng.dialect, tm.model_id, tm.config.arch).cross_check(tm.config.arch)
    if warn:
        print(f"[r4dxb-server] warning: {warn}", file=sys.stderr)
    audio_id = -1
    if getattr(args, "audio", "off") == "on" and args.batch <= 1:
        from ..models.audio import load_audio_embedder
        eng.audio = load_audio_embedder(getattr(tm.m, "w", {}))
        audio_id = getattr(tk, "audio_token_id", tm.config.vocab_size - 2)
    defaults = {"temperature": args.default_temperature, "top_k": args.default_top_k, "top_p": args.default_top_p,
                "min_p": args.default_min_p, "repetition_penalty": args.default_repetition_penalty}
    srv = ApiServer(eng, tk, tpl, tm.model_id, host=args.host, port=args.port, max_tokens_default=args.max_tokens_default,
                    defaults=defaults, spec_k=args.mtp or getattr(args, "ngram", 0), vision_config=vcfg, image_token_id=image_id, audio_token_id=audio_id)
    print(f"[r4dxb-server] {tm.model_id} on http://{args.host}:{srv.port} (tp={tm.tp_world()})", file=sys.stderr)
    try:
        srv.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        eng.shutdown()
        if hasattr(tm, "shutdown"):
            tm.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
