"""The command line, in the manner of the reference's `burn-lm-cli` (crates/burn-lm-cli/src/cli.rs:
5-69): `models`, `run <model> [flags] <prompt> [--no-stats]` (commands/run.rs:7-97), `chat <model>`
with /help /stats /clear /exit (commands/chat.rs:13-211) and `shell`, the default, which offers the
same commands without the program's name (commands/shell.rs:27-184).  Flags are the reference's
per-request options: --top-p, --temperature, --max-seq-len, --sample-len, --seed
(crates/burn-lm-llama/src/server/llama3.rs:14-31).

A model is a folder (config.json, model.safetensors).  There is no tokenizer here: a prompt is
either a list of token ids ("12,7,99" or "12 7 99") or text, which is read as bytes, one token per
byte, like the reference's ByteTokenizer (crates/burn-lm-llama/src/tokenizer/byte.rs:14-36; needs a
vocabulary of at least 256).  `random` writes a model folder with random weights from a config.json or a named preset.
"""
from __future__ import annotations

import argparse
import json
import re
import shlex
import sys

from . import api
from .registry import architectures


def parse_prompt(text: str, vocab: int):
    """(token ids, was_text)."""
    if re.fullmatch(r"\s*\d+(?:[\s,]+\d+)*\s*", text):
        return [int(t) for t in re.split(r"[\s,]+", text.strip())], False
    if vocab < 256:
        raise SystemExit(f"a text prompt is read as bytes and needs a vocabulary of 256 or more; this model has {vocab}")
    return list(text.encode("utf-8")), True


def render(tokens, as_text: bool) -> str:
    if as_text and all(0 <= t < 256 for t in tokens):
        return bytes(tokens).decode("utf-8", errors="replace")
    return " ".join(str(t) for t in tokens)


def stats_table(out, load_seconds: float) -> str:
    s = out.stats
    rows = [("inference duration", f"{s.inference_seconds:.3f} s"),
            ("  prefill", f"{s.prefill_seconds:.3f} s for {s.prompt_tokens} tokens"),
            ("  decode", f"{s.decode_seconds:.3f} s for {s.decode_steps} steps"),
            ("tokens count", str(s.generated_tokens)),
            ("tokens per second", f"{s.tokens_per_second:.1f}"),
            ("model loading duration", f"{load_seconds:.3f} s"),
            ("total duration", f"{s.inference_seconds + load_seconds:.3f} s"),
            ("seed", str(s.seed))]
    w = max(len(r[0]) for r in rows)
    return "\n".join(["| " + "Stat".ljust(w) + " | Value", "|-" + "-" * w + "-|------"] +
                     [f"| {k.ljust(w)} | {v}" for k, v in rows])


def add_request_flags(p):
    p.add_argument("--top-p", type=float, default=0.9, help="Top-p probability threshold.")
    p.add_argument("--temperature", type=float, default=0.0,
                   help="Temperature value for controlling randomness in sampling.")
    p.add_argument("--max-seq-len", type=int, default=8192, help="Maximum sequence length for input text.")
    p.add_argument("--sample-len", type=int, default=4096, help="The number of new tokens to generate.")
    p.add_argument("--seed", type=int, default=0,
                   help="The seed to use when generating random samples. If it is 0 then a random seed is used.")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="Compute dtype.")
    p.add_argument("--include-stop", action="store_true", help="Print the stop token that ended the answer as well.")


def build_parser(prog="burn-lm"):
    ap = argparse.ArgumentParser(prog=prog, description="B200-native generation with the dense Llama decoder")
    sub = ap.add_subparsers(dest="command")
    sub.add_parser("models", help="List the registered architectures")
    run = sub.add_parser("run", help="Run inference on a model folder in the terminal")
    run.add_argument("model", help="model folder (config.json, model.safetensors)")
    add_request_flags(run)
    run.add_argument("--no-stats", action="store_true", help="Disable display of statistics at the end of the inference")
    run.add_argument("prompt", help="The prompt to send to the model: token ids, or text read as bytes")
    chat = sub.add_parser("chat", help="Start a chat session with a model folder")
    chat.add_argument("model")
    add_request_flags(chat)
    rnd = sub.add_parser("random", help="Write a model folder with random weights")
    rnd.add_argument("folder", help="where to write config.json and model.safetensors")
    src = rnd.add_mutually_exclusive_group(required=True)
    src.add_argument("--config", help="a config.json to take the sizes from")
    src.add_argument("--preset", help="a named configuration (see `models`)")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    sub.add_parser("shell", help="Start a shell in which the commands run without the program's name (default)")
    return ap


def cmd_models(_args):
    print("| Architecture | Description")
    print("|--------------|------------")
    for a in architectures():
        print(f"| {a.name} | {a.description}")
    from .config import preset_names
    print("presets for `random --preset`: " + ", ".join(preset_names()))


def cmd_random(args):
    from .config import preset
    from .weights import write_random_model
    if args.preset:
        cfg = preset(args.preset)
    else:
        with open(args.config) as f:
            cfg = json.load(f)
    write_random_model(args.folder, cfg, args.seed, args.dtype)
    print(f"wrote {args.folder}")


def _load(args):
    print(f"loading model '{args.model}'...", file=sys.stderr)
    lm = api.load(args.model, dtype=args.dtype, max_seq_len=args.max_seq_len, max_batch=1)
    print("model loaded!", file=sys.stderr)
    return lm


def _answer(lm, args, prompt_text, show_stats):
    tokens, as_text = parse_prompt(prompt_text, lm.engine.vocab_size)
    out = lm.generate([tokens], temperature=args.temperature, top_p=args.top_p, sample_len=args.sample_len,
                      seed=args.seed, include_stop=args.include_stop)
    r = out.results[0]
    if r.error is not None:
        print(f"An error occurred: {r.error}", file=sys.stderr)
        return 1
    print("\n" + render(r.tokens, as_text))
    if show_stats:
        print(stats_table(out, lm.load_seconds))
    return 0


def cmd_run(args):
    lm = _load(args)
    rc = _answer(lm, args, args.prompt, not args.no_stats)
    lm.unload()
    return rc


CHAT_HELP = "/help  show this help\n/stats  toggle statistics\n/clear  clear the state\n/exit  leave the chat"


def cmd_chat(args, stdin=None):
    lm = _load(args)
    stdin = stdin or sys.stdin
    show_stats = True
    print("Chat session started! (/help for commands)")
    while True:
        print("> ", end="", flush=True)
        line = stdin.readline()
        if not line:
            break
        line = line.strip()
        if not line:
            continue
        if line.startswith("/"):
            word = line.split()[0]
            if word == "/exit":
                break
            if word == "/help":
                print(CHAT_HELP)
            elif word == "/stats":
                show_stats = not show_stats
                print(f"stats {'on' if show_stats else 'off'}")
            elif word == "/clear":
                lm.clear_state()
                print("state cleared")
            else:
                print(f"unknown command {word}; {CHAT_HELP}")
            continue
        _answer(lm, args, line, show_stats)
    lm.unload()
    return 0


def cmd_shell(_args, stdin=None):
    stdin = stdin or sys.stdin
    parser = build_parser(prog="")
    while True:
        print("(b200) burnlm> ", end="", flush=True)
        line = stdin.readline()
        if not line:
            break
        line = line.strip()
        if line in ("exit", "quit"):
            break
        if not line:
            continue
        try:
            args = parser.parse_args(shlex.split(line))
        except SystemExit:
            continue
        if args.command in (None, "shell"):
            parser.print_help()
            continue
        try:
            dispatch(args, stdin)
        except SystemExit as e:
            print(e, file=sys.stderr)
        except Exception as e:  # a failed command does not end the shell
            print(f"An error occurred: {e}", file=sys.stderr)
    return 0


def dispatch(args, stdin=None):
    if args.command == "models":
        return cmd_models(args)
    if args.command == "run":
        return cmd_run(args)
    if args.command == "chat":
        return cmd_chat(args, stdin)
    if args.command == "random":
        return cmd_random(args)
    return cmd_shell(args, stdin)


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return dispatch(args) or 0
