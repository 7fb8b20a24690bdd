"""`colossalai_b200 replay`: feed given token ids through a served model step by step and write the logits asked for.

Nothing is sampled.  Each line of standard input is one engine step,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

whose entries - portions of prompts beside single tokens - run as ONE ragged batch through `LLMEngine.forward_ragged`,
the step function of the engine's own generation loop, on the engine's page pool and state slots.  A request is admitted
at its first entry and gives its pages and slot back when a step lists it under "end".  A step that asks for logits
writes `<out>/<step>.f32` (little-endian fp32, [wanted rows, vocab], in the order of the entries and of "want"); every
step answers `done <step>` on standard output.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

__all__ = ["add_replay_parser", "replay"]


def replay(model: str, dtype: str, out_dir: str, max_tokens: int, stream_in=None, stream_out=None, max_live: int = 4,
           block_size: int = 16) -> int:
    import torch

    from ...inference.config import InferenceConfig
    from ...inference.core.llm_engine import LLMEngine
    from ...inference.struct import Sequence

    stream_in = stream_in or sys.stdin
    stream_out = stream_out or sys.stdout
    tdtype = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[dtype]
    if tdtype == torch.float32:                        # true 32-bit products, no reduced-precision matrix mode
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        torch.set_float32_matmul_precision("highest")
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    max_tokens = (max_tokens + block_size - 1) // block_size * block_size
    cfg = InferenceConfig(dtype=tdtype, max_batch_size=max_live, max_input_len=max_tokens, max_output_len=block_size,
                          block_size=block_size, max_cache_tokens=max_tokens, max_num_batched_tokens=max_tokens,
                          enable_chunked_prefill=True, use_cuda_graph=False)
    engine = LLMEngine(model, inference_config=cfg)
    handler = engine.request_handler
    os.makedirs(out_dir, exist_ok=True)
    for line in stream_in:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries, want = [], []
        for e in step.get("entries", []):
            rs = handler.live.get(e["id"])
            if rs is None:
                rs = handler.admit(Sequence(e["id"], None, [], block_size, None, -1, 0, max_output_len=1 << 30,
                                            ignore_eos=True))
            rs.seq.input_token_id += list(e["tokens"])
            entries.append((rs, e["tokens"]))
            want.append(list(e.get("want", [])))
        if any(len(toks) for _, toks in entries):
            logits = engine.forward_ragged(entries, want)
            if logits.shape[0]:
                data = logits.float().cpu().contiguous().numpy().astype("<f4")
                tmp = os.path.join(out_dir, f".{step['step']}.part")
                with open(tmp, "wb") as f:
                    f.write(data.tobytes())
                os.replace(tmp, os.path.join(out_dir, f"{step['step']}.f32"))
        for rid in step.get("end", []):
            if rid in handler.live:
                handler.release(rid)
        stream_out.write(f"done {step['step']}\n")
        stream_out.flush()
    return 0


def _run(args: argparse.Namespace, extra) -> int:
    return replay(args.model, args.dtype, args.out, args.max_tokens, max_live=args.max_live)


def add_replay_parser(sub) -> None:
    p = sub.add_parser("replay", help="replay a trace of token ids through the serving engine and write logits")
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    p.add_argument("--out", required=True, help="folder for <step>.f32")
    p.add_argument("--max-tokens", type=int, required=True, help="tokens that live requests hold at any time")
    p.add_argument("--max-live", type=int, default=4, help="state slots (requests live at once)")
    p.set_defaults(func=_run)
