"""Command line: ``python -m rosellm_b200.cli_generate --model DIR --prompt TEXT``.

Options keep the names and meanings of the reference's
``python -m rosellm.roseinfer.cli_generate`` (rosellm/roseinfer/cli_generate.py:21-139):
``--prompt``, ``--interactive``, ``--system-prompt``, ``--max-new-tokens`` (100),
``--top-k`` (0), ``--top-p`` (1.0), ``--temperature`` (1.0), ``--stop-on-eos`` /
``--no-stop-on-eos``, ``--do-sample``, ``--device``, ``--no-amp`` (32-bit), ``--bf16``,
``--stream``, ``--tokenizer-name``.  The model comes from a local folder
(``--model``; ``--checkpoint-path`` and ``--hf-model-id`` are accepted as other names
for it, there being no network and no training checkpoints here), or has random
weights (``--random-weights CONFIG.json --seed S``).  ``--prompt-ids`` (or
``--prompt-ids-file``, a file of ids separated by commas or white space) gives the prompt
as token ids, for folders without a tokenizer; ids then come out as well.  The engine's own
options: ``--dtype`` (``bf16`` or ``fp32``; ``--no-amp`` means ``fp32``), ``--page-size``,
the cache's size as ``--num-pages``, ``--kv-cache-max-tokens`` or
``--gpu-memory-utilization``, ``--max-num-seqs`` (the reference's ``--max-batch-size``),
``--max-num-batched-tokens`` and ``--prefill-chunk-size``.
"""
from __future__ import annotations

import argparse
import json
import sys

ROLE_SYSTEM, ROLE_USER, ROLE_ASSISTANT = "System", "User", "Assistant"
EXIT_COMMANDS = {"/exit", "/quit"}
CLEAR_COMMAND = "/clear"


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Generate text from a model")
    p.add_argument("--model", "--checkpoint-path", "--hf-model-id", dest="model", default=None,
                   help="folder with config.json and model.safetensors")
    p.add_argument("--random-weights", default=None, metavar="CONFIG_JSON",
                   help="no weight file: a config.json whose model gets random weights")
    p.add_argument("--seed", type=int, default=0, help="seed of the random weights and of sampling")
    p.add_argument("--tokenizer-name", default=None, help="folder of a tokenizer (default: the model folder)")
    p.add_argument("--prompt", default=None, help="Prompt to generate text from")
    p.add_argument("--prompt-ids", default=None, help="prompt as comma-separated token ids")
    p.add_argument("--prompt-ids-file", default=None, metavar="FILE",
                   help="file with the prompt's token ids, separated by commas or white space")
    p.add_argument("--interactive", action="store_true", help="Run interactive multi-turn chat in the shell")
    p.add_argument("--system-prompt", default="", help="Optional system instruction used in interactive mode")
    p.add_argument("--max-new-tokens", type=int, default=100, help="Maximum number of new tokens to generate")
    p.add_argument("--top-k", type=int, default=0, help="Top-k sampling")
    p.add_argument("--top-p", type=float, default=1.0, help="Top-p sampling")
    p.add_argument("--temperature", type=float, default=1.0, help="Temperature for sampling")
    p.add_argument("--stop-on-eos", dest="stop_on_eos", action="store_true", help="Stop on EOS token")
    p.add_argument("--no-stop-on-eos", dest="stop_on_eos", action="store_false", help="Do not stop on EOS token")
    p.set_defaults(stop_on_eos=True)
    p.add_argument("--do-sample", action="store_true", help="Use sampling to generate text (or else greedy)")
    p.add_argument("--device", default="cuda", help="Device to use")
    p.add_argument("--no-amp", action="store_true", help="Run everything in 32-bit")
    p.add_argument("--bf16", action="store_true", help="Use bfloat16 (the only 16-bit path here)")
    p.add_argument("--stream", action="store_true", help="Stream the output")
    p.add_argument("--dtype", default=None, choices=["bf16", "bfloat16", "fp32", "float32"],
                   help="precision of the whole model (default: bf16, or fp32 with --no-amp)")
    p.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    p.add_argument("--num-pages", type=int, default=None, help="pages the cache holds")
    p.add_argument("--kv-cache-max-tokens", type=int, default=None, help="tokens the cache holds")
    p.add_argument("--gpu-memory-utilization", type=float, default=None,
                   help="share of the device the engine may fill; the cache gets what the weights leave of it")
    p.add_argument("--max-num-seqs", "--max-batch-size", dest="max_num_seqs", type=int, default=8,
                   help="requests in flight at most")
    p.add_argument("--max-num-batched-tokens", type=int, default=2048, help="tokens one step runs at most")
    p.add_argument("--prefill-chunk-size", type=int, default=512, help="longest prompt portion per step")
    args = p.parse_args(argv)
    if args.model is None and args.random_weights is None:
        p.error("--model (or --random-weights CONFIG.json) is required")
    if sum(v is not None for v in (args.prompt_ids, args.prompt_ids_file)) > 1:
        p.error("give --prompt-ids or --prompt-ids-file, not both")
    if not args.interactive and args.prompt is None and args.prompt_ids is None and args.prompt_ids_file is None:
        p.error("--prompt (or --prompt-ids, --prompt-ids-file) is required unless --interactive is enabled.")
    if args.dtype is not None and args.no_amp and args.dtype in ("bf16", "bfloat16"):
        p.error("--no-amp asks for 32-bit and --dtype for bfloat16")
    return args


def prompt_ids_of(args) -> list[int] | None:
    """The prompt as token ids, when it was given so (``--prompt-ids`` or ``--prompt-ids-file``)."""
    text = args.prompt_ids
    if args.prompt_ids_file is not None:
        with open(args.prompt_ids_file, encoding="utf-8") as f:
            text = f.read()
    if text is None:
        return None
    return [int(t) for t in text.replace(",", " ").split()]


INDENT = "  "


def _section(role: str, text: str) -> list[str]:
    return [f"{role}:"] + [INDENT + line for line in (str(text).splitlines() or [""])]


def build_chat_prompt(system_prompt: str, history: list[tuple[str, str]], user_input: str) -> str:
    """The chat template of rosellm/roseinfer/cli_generate.py:140-163: a ``System:`` section when
    there is a system prompt, a ``User:`` / ``Assistant:`` section pair per earlier turn, the new
    ``User:`` section and an open ``Assistant:`` section; the text of a section is indented by
    two spaces under its header."""
    lines: list[str] = []
    if system_prompt:
        lines += _section(ROLE_SYSTEM, system_prompt)
    for user_text, assistant_text in history:
        lines += _section(ROLE_USER, user_text) + _section(ROLE_ASSISTANT, assistant_text)
    lines += _section(ROLE_USER, user_input)
    lines += [f"{ROLE_ASSISTANT}:", INDENT]
    return "\n".join(lines)


def clean_reply(generated: str) -> str:
    """What of a generated continuation is the assistant's turn: lines up to the first that
    opens a ``User:`` or ``System:`` section, a leading ``Assistant:`` removed
    (rosellm/roseinfer/cli_generate.py:166-236)."""
    kept: list[str] = []
    for raw in generated.split("\n"):
        if raw.startswith(f"{ROLE_USER}:") or raw.startswith(f"{ROLE_SYSTEM}:"):
            break
        line = raw[len(ROLE_ASSISTANT) + 1:].lstrip() if raw.startswith(f"{ROLE_ASSISTANT}:") else raw
        if not kept:
            line = line.lstrip()
            if not line:
                continue
        kept.append(line)
    return "\n".join(kept).rstrip()


def run_interactive(engine, args, read=input, write=print) -> None:
    """A chat loop in the shell: ``/clear`` forgets the history, ``/exit`` and ``/quit`` leave;
    ``--prompt``, when given, is the first user turn (rosellm/roseinfer/cli_generate.py:239-301)."""
    write("[rosellm_b200] interactive mode enabled")
    write(f"[rosellm_b200] commands: {CLEAR_COMMAND} {' '.join(sorted(EXIT_COMMANDS))}")
    history: list[tuple[str, str]] = []
    first = (args.prompt or "").strip()
    while True:
        if first:
            user_input, first = first, ""
            write(f"You> {user_input}")
        else:
            try:
                user_input = read("You> ").strip()
            except (EOFError, KeyboardInterrupt):
                write("[rosellm_b200] exiting interactive mode.")
                return
        if not user_input:
            continue
        if user_input in EXIT_COMMANDS:
            write("[rosellm_b200] exiting interactive mode.")
            return
        if user_input == CLEAR_COMMAND:
            history.clear()
            write("[rosellm_b200] chat history cleared.")
            continue
        prompt = build_chat_prompt(args.system_prompt, history, user_input)
        reply = clean_reply(engine.generate(
            prompt, max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_k=args.top_k,
            top_p=args.top_p, stop_on_eos=args.stop_on_eos, do_sample=args.do_sample, seed=args.seed))
        write(f"Assistant> {reply}")
        history.append((user_input, reply))


def make_engine(args):
    from .engine.llm import InferenceEngine

    common = dict(device=args.device, use_amp=not args.no_amp, bf16=True, dtype=args.dtype,
                  tokenizer_name=args.tokenizer_name, page_size=args.page_size, num_pages=args.num_pages,
                  kv_cache_max_tokens=args.kv_cache_max_tokens, gpu_memory_utilization=args.gpu_memory_utilization,
                  max_batch_size=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens,
                  prefill_chunk_size=args.prefill_chunk_size, sampling_seed=args.seed)
    if args.model is not None:
        return InferenceEngine(args.model, **common)
    from .config.base import parse_config

    with open(args.random_weights) as f:
        config = parse_config(json.load(f))
    return InferenceEngine(config=config, seed=args.seed, **common)


def main(argv=None) -> int:
    args = parse_args(argv)
    engine = make_engine(args)
    print(f"[rosellm_b200] device: {engine.device}")
    print(f"[rosellm_b200] use_amp: {engine.use_amp}")
    if args.interactive:
        run_interactive(engine, args)
        return 0
    kw = dict(max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_k=args.top_k,
              top_p=args.top_p, stop_on_eos=args.stop_on_eos, do_sample=args.do_sample, seed=args.seed)
    ids = prompt_ids_of(args)
    prompt = args.prompt if ids is None else ids
    print(f"[rosellm_b200] prompt: {prompt}")
    if args.stream:
        print("[rosellm_b200] streaming output: ", end="", flush=True)
        for piece in engine.stream_generate(prompt, **kw):
            print(piece if isinstance(piece, str) else f"{piece} ", end="", flush=True)
        print()
    else:
        print(f"[rosellm_b200] output: {engine.generate(prompt, **kw)}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
