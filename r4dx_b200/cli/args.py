"""Flag definitions shared by the CLI generator and the server (reference: src/cli/cli_args.h,
src/server/server_args.h; flag names follow the reference's so scripts carry over)."""
from __future__ import annotations

import argparse
import os


def add_model_flags(ap: argparse.ArgumentParser) -> None:
    g = ap.add_argument_group("model")
    g.add_argument("--model", required=False, help="container file (.r4dxb) or 'synthetic:<tiny|small|27b>'")
    g.add_argument("--layout", default="trellis", choices=["bf16", "w4a16", "trellis", "w8a16"])
    g.add_argument("--tokenizer-dir", default=None)
    g.add_argument("--max-ctx", type=int, default=8192)
    g.add_argument("--layers", type=int, default=0, help="load only the first N layers (debug)")
    g.add_argument("--prefill-chunk", type=int, default=int(os.environ.get("R4DXB_PREFILL_CHUNK", "0")),
                   help="rows per prefill chunk (0: chosen from the prompt length)")
    g.add_argument("--mtp", type=int, default=0, metavar="K", help="MTP speculative decoding with K drafts per round")
    g.add_argument("--ngram", type=int, default=0, metavar="K",
                   help="n-gram (prompt-lookup) speculative decoding with up to K drafts per round; needs no drafter weights")
    g.add_argument("--dflash", default=None, metavar="CONTAINER", help="block-diffusion drafter container")
    g.add_argument("--dflash-k", type=int, default=7)
    g.add_argument("--dflash-p-min", type=float, default=0.0)
    g.add_argument("--dflash-n-min", type=int, default=0)
    g.add_argument("--vision", default="off", choices=["off", "on"])
    g.add_argument("--image-max-pixels", type=int, default=0,
                   help="upper bound on an image's resized area in pixels (0: the vision tower's own limit); the hybrid family's tower")
    g.add_argument("--image-soft-tokens", type=int, default=0,
                   help="rows an image may take in the prompt (70, 140, 280, 560 or 1120; 0: 280); the Gemma-style family's embedder")
    g.add_argument("--mtp-draft-head", default="on", choices=["on", "off"],
                   help="use the container's reduced-vocabulary draft head for the MTP drafter's own drafts when it has one")
    g.add_argument("--ngram-sidecar", default=None, metavar="FILE",
                   help="qwen4_exp: the n-gram table file (default: the one the container records, next to it)")
    g.add_argument("--ngram-placement", default="device", choices=["device", "pinned", "file"],
                   help="qwen4_exp: where the n-gram table lives; device (95 GiB for the full table, no host work per token, "
                        "CUDA-graph decode), pinned host memory, or positioned reads from the file (both: host ids, eager decode)")
    g.add_argument("--dialect", default="auto", choices=["auto", "qwen", "gemma", "lfm2", "llama", "qwen4_exp"],
                   help="reasoning markers and tool-call syntax; auto picks by model id and architecture")
    g.add_argument("--audio", default="off", choices=["off", "on"],
                   help="accept input_audio parts (the container must hold the audio projection; Gemma-style family)")
    p = ap.add_argument_group("parallelism")
    p.add_argument("--tp", type=int, default=1, choices=[1, 2, 4, 8])
    p.add_argument("--tp-mode", default=os.environ.get("R4DXB_TP_MODE", "fused"), choices=["fused", "nccl", "noop"])
    p.add_argument("--tp-ar-timeout-ms", type=int, default=500)
    p.add_argument("--pp", type=int, default=1, choices=[1, 2])
    p.add_argument("--pp-split", type=int, default=0, help="first layer of the second stage (0: chosen by --pp-balance)")
    p.add_argument("--pp-balance", default="layers", choices=["layers", "bytes"],
                   help="how --pp-split 0 places the boundary: by layer count (equal prefill work, the head counted with the "
                        "second stage) or by weight bytes (models that only fit when the two devices hold equal shares)")
    p.add_argument("--pp-min-rows", type=int, default=512)
    p.add_argument("--ep", type=int, default=1, choices=[1, 2, 4, 8],
                   help="expert parallelism for mixture-of-experts models: whole attention per rank, a slice of the experts each")
    p.add_argument("--hybrid-ctx", type=int, default=0,
                   help="--hybrid: positions the two pipeline stages keep state for (0: --max-ctx); longer prompts prefill tensor-parallel")
    p.add_argument("--hybrid", action="store_true", help="pipeline-parallel prefill, then reshard to tensor-parallel decode")
    p.add_argument("--tp-fault", default=os.environ.get("R4DXB_TP_FAULT", ""), help="host-side fault injection 'rank:n:kind'")


def add_sampling_flags(ap: argparse.ArgumentParser, prefix: str = "") -> None:
    g = ap.add_argument_group("sampling")
    g.add_argument(f"--{prefix}temperature", type=float, default=0.0 if not prefix else 1.0)
    g.add_argument(f"--{prefix}top-k", type=int, default=0)
    g.add_argument(f"--{prefix}top-p", type=float, default=1.0)
    g.add_argument(f"--{prefix}min-p", type=float, default=0.0)
    g.add_argument(f"--{prefix}repetition-penalty", type=float, default=1.0)


def cli_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser("r4dxb-cli", description="one-shot / chat text generation")
    add_model_flags(ap)
    add_sampling_flags(ap)
    ap.add_argument("--prompt", default=None)
    ap.add_argument("--prompt-file", default=None)
    ap.add_argument("--system", default=None)
    ap.add_argument("--chat", action="store_true")
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--think", default="on", choices=["on", "off"])
    ap.add_argument("--stats", action="store_true")
    ap.add_argument("--profile", action="store_true", help="per-op device timing of one decode step")
    ap.add_argument("--profile-prefill", action="store_true")
    ap.add_argument("--dump-token-ids", action="store_true")
    ap.add_argument("--image", action="append", default=[], metavar="FILE",
                    help="image file placed before the prompt text (repeatable); needs --vision on")
    return ap


def server_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser("r4dxb-server", description="OpenAI-compatible server")
    add_model_flags(ap)
    add_sampling_flags(ap, "default-")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--max-queue", type=int, default=8)
    ap.add_argument("--max-tokens-default", type=int, default=512)
    ap.add_argument("--log-level", default="info", choices=["debug", "info", "warn", "error"])
    ap.add_argument("--prompt-checkpoint", default="on", choices=["on", "off"])
    ap.add_argument("--request-log", default=None)
    ap.add_argument("--request-log-tokens", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="concurrent decode slots")
    ap.add_argument("--batch-ctx", type=int, default=32768)
    return ap


def convert_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser("r4dxb-convert", description="checkpoint -> quantized container")
    ap.add_argument("--input", default=None, help="safetensors file/dir with config.json, a .gguf file, or 'random:<tiny|small|moe|llama|gemma|lfm2|q4x>'")
    ap.add_argument("--output", default=None)
    ap.add_argument("--layouts", default="trellis", help="body layout: trellis, w4a16, w8a16 or bf16")
    ap.add_argument("--lm-head", default="w4a16", choices=["w4a16", "bf16"])
    ap.add_argument("--lm-head-group", type=int, default=64)
    ap.add_argument("--kb-plan", default="mix4.5", choices=["mix4.5", "mix3.3", "kb3", "kb4", "kb5"])
    ap.add_argument("--kb-plan-file", default=None, metavar="PLAN.json",
                    help="per-class trellis bit widths written by `python -m r4dx_b200.utils.alloc_bits` (classes it does not "
                         "name take --kb-plan)")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--threads", type=int, default=0)
    ap.add_argument("--encoder", default="cpu", choices=["cpu", "cuda"], help="where the trellis Viterbi search runs")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--mtp", action="store_true")
    ap.add_argument("--keep-bf16", default="", help="comma list of tensor-name substrings kept in bf16")
    ap.add_argument("--hessians", default=None,
                    help="safetensors file from `python -m r4dx_b200.quant.calibrate hessians`: linears found in it are quantized "
                         "with error compensation (block LDLQ for trellis, GPTQ for w4a16)")
    ap.add_argument("--quant", default="rtn", choices=["rtn", "search"],
                    help="w4a16 layout: round to nearest over the full group range, or search the clipping range per group")
    ap.add_argument("--imatrix", default=None,
                    help="safetensors file from `python -m r4dx_b200.quant.calibrate imatrix`: weighs the search by channel importance")
    ap.add_argument("--kv-calib", default=None, help="JSON file with per-layer k/v amax for fp8 descales")
    ap.add_argument("--reuse-tensors-from", default=None, help="older container whose identical tensors are copied, guarded by sha256")
    ap.add_argument("--rotate", default="none", choices=["none", "q2a", "q2ab"],
                    help="residual-stream rotation folded into the weights before quantization (dense hybrid family); "
                         "q2ab equals q2a for trellis bodies, whose linears already carry their own block Hadamards")
    ap.add_argument("--rotation-seed", type=lambda v: int(v, 0), default=0x5EED, help="u64, decimal or 0x hex")
    ap.add_argument("--rotation-block", type=int, default=0, help="Hadamard block of the rotation (default: up to 1024)")
    ap.add_argument("--rotation-out", default=None, metavar="FILE.safetensors",
                    help="with --rotate and no quantization wanted: write only the rotation tensors and exit")
    ap.add_argument("--vision", default="off", choices=["on", "off"], help="keep the checkpoint's vision tower tensors (bf16)")
    ap.add_argument("--audio", default="off", choices=["on", "off"],
                    help="keep the checkpoint's audio embedder tensors ([model.]embed_audio.* -> audio.embed_audio.*, bf16; Gemma-style family)")
    ap.add_argument("--ngram-sidecar", default=None, metavar="FILE",
                    help="qwen4_exp: the n-gram table file the container refers to (required for that family; a random:q4x source "
                         "writes a small synthetic table there if the file does not exist)")
    ap.add_argument("--dflash-hf", default=None, metavar="DIR",
                    help="also convert a block-diffusion drafter checkpoint (safetensors + config.json) into <output>.dflash")
    ap.add_argument("--trellis-from", default=None, metavar="DIR",
                    help="import already-encoded trellis tensors (<name>.trellis.words/.suh/.svh in safetensors files of DIR, "
                         "this engine's tile order) instead of encoding those linears; every imported tensor is reconstructed on "
                         "the CPU and checked against the checkpoint")
    ap.add_argument("--trellis-verify", default="full", choices=["full", "none"])
    ap.add_argument("--w4a16-group-rule", default="", metavar="REGEX=GROUP[,REGEX=GROUP...]",
                    help="w4a16 group size per tensor name, first match wins (e.g. '^lm_head$=32'); others use --lm-head-group")
    ap.add_argument("--w8a16-group", type=int, default=0, help="group size of the w8a16 body layout (default: --lm-head-group)")
    ap.add_argument("--ldlq-damp", type=float, default=0.01, help="relative diagonal damping of the Hessians in the error-compensated trellis quantizer")
    ap.add_argument("--trellis-manifest-sha256", default=None, metavar="HEX",
                    help="with --trellis-from: refuse the directory unless its trellis_manifest.json has this sha256")
    ap.add_argument("--draft-vocab-ids", default=None, metavar="FILE.json",
                    help="with --mtp: a JSON list of token ids (or {\"ids\": [...]}); the container gets a smaller head over those "
                         "ids (mtp.draft_head.lm_head + mtp.draft_head.vocab_ids) that the MTP drafter uses for its own drafts")
    ap.add_argument("--plan-only", action="store_true",
                    help="plan every tensor (layout, bit width, bytes) and print the container's tensor count and data bytes "
                         "without quantizing anything or writing --output")
    ap.add_argument("--selftest-input", default=None, metavar="FILE.safetensors",
                    help="one-tensor self test: quantize the 2-D tensor \"w\" of this file as if it were named --selftest-name, "
                         "reconstruct it, print the error (and write the reconstruction to --selftest-output); needs no --input / --output")
    ap.add_argument("--selftest-name", default="text.layers.0.mlp.down")
    ap.add_argument("--selftest-output", default=None, metavar="FILE.safetensors")
    ap.add_argument("--selftest", action="store_true", help="re-open the output and verify every tensor's reconstruction error")
    return ap
