"""The command line's own decisions, with a stand-in for the loaded model: prompt parsing, rendering, the
statistics table, `run`, the `chat` commands and the `shell`, whose failing commands must not end it.
(reference: crates/burn-lm-cli/src/commands/run.rs:7-97, commands/chat.rs:140-195, commands/shell.rs:136-181)"""
import io
import json
import os

import pytest

from burn_lm_b200 import cli
from burn_lm_b200.cache import ContextLengthExceeded
from burn_lm_b200.engine.generate import GenerationOutput, GenerationStats, RequestResult


class StandIn:
    """What the command line asks of a loaded model."""

    def __init__(self, vocab=300):
        self.calls, self.cleared, self.unloaded = [], 0, 0
        self.load_seconds = 0.25
        self.engine = type("E", (), {"vocab_size": vocab})()

    def generate(self, prompts, **options):
        self.calls.append((prompts, options))
        p = prompts[0]
        if len(p) > 20:
            return GenerationOutput([RequestResult(finish_reason="error", error=ContextLengthExceeded(len(p), 20))], GenerationStats())
        answer = [t + 1 for t in p][: options["sample_len"]]
        stats = GenerationStats(prompt_tokens=len(p), generated_tokens=len(answer), prefill_seconds=0.5, decode_seconds=1.5,
                                decode_steps=len(answer), batches=1, seed=options["seed"] or 99)
        return GenerationOutput([RequestResult(tokens=answer, finish_reason="length", prompt_tokens=len(p))], stats)

    def clear_state(self):
        self.cleared += 1

    def unload(self):
        self.unloaded += 1


@pytest.fixture
def model(monkeypatch):
    lm = StandIn()
    loads = []
    monkeypatch.setattr(cli.api, "load", lambda folder, **kw: (loads.append((folder, kw)), lm)[1])
    lm.loads = loads
    return lm


def test_parse_prompt_and_render():
    assert cli.parse_prompt("12,7, 99", 300) == ([12, 7, 99], False)
    assert cli.parse_prompt(" 5 6\t7 ", 300) == ([5, 6, 7], False)
    assert cli.parse_prompt("hé", 300) == (list("hé".encode()), True)
    with pytest.raises(SystemExit, match="256"):
        cli.parse_prompt("words", 255)
    assert cli.render([104, 105], True) == "hi"
    assert cli.render([104, 300], True) == "104 300"        # not bytes: shown as ids
    assert cli.render([1, 2], False) == "1 2"


def test_stats_table():
    stats = GenerationStats(prompt_tokens=7, generated_tokens=30, prefill_seconds=0.5, decode_seconds=1.5, decode_steps=29, seed=4)
    table = cli.stats_table(GenerationOutput([], stats), 0.25)
    lines = table.splitlines()
    assert lines[0].startswith("| Stat") and set(lines[1]) <= set("|- ")
    text = "\n".join(lines)
    for needle in ("2.000 s", "0.500 s for 7 tokens", "1.500 s for 29 steps", "| 30", "15.0", "0.250 s", "2.250 s", "| 4"):
        assert needle in text, needle


def test_run_passes_the_reference_options(model, capsys):
    rc = cli.main(["run", "some/folder", "--temperature", "0.7", "--top-p", "0.5", "--sample-len", "3", "--seed", "11",
                   "--max-seq-len", "512", "--dtype", "float32", "4 5 6 7"])
    assert rc == 0
    folder, kw = model.loads[0]
    assert folder == "some/folder" and kw == {"dtype": "float32", "max_seq_len": 512, "max_batch": 1}
    prompts, options = model.calls[0]
    assert prompts == [[4, 5, 6, 7]]
    assert options == {"temperature": 0.7, "top_p": 0.5, "sample_len": 3, "seed": 11, "include_stop": False}
    out = capsys.readouterr().out
    assert "5 6 7" in out and "tokens per second" in out and model.unloaded == 1
    # defaults are the reference's: top_p 0.9, temperature 0, sample_len 4096, seed 0, max_seq_len 8192
    cli.main(["run", "m", "--no-stats", "hi"])
    assert model.loads[1][1]["max_seq_len"] == 8192
    assert model.calls[1][1] == {"temperature": 0.0, "top_p": 0.9, "sample_len": 4096, "seed": 0, "include_stop": False}
    out = capsys.readouterr().out
    assert "ij" in out and "tokens per second" not in out           # text in, text out; no table


def test_run_reports_a_request_error(model, capsys):
    rc = cli.main(["run", "m", " ".join(["1"] * 30)])
    assert rc == 1
    assert "exceeds the maximum of 20" in capsys.readouterr().err


def test_chat_commands(model, capsys):
    stdin = io.StringIO("/help\n1 2\n/stats\n3\n/nonsense\n\n/clear\n/exit\n9 9 9\n")
    args = cli.build_parser().parse_args(["chat", "m", "--sample-len", "5"])
    assert cli.dispatch(args, stdin) == 0
    out = capsys.readouterr().out
    assert "/stats  toggle statistics" in out and "stats off" in out and "unknown command /nonsense" in out and "state cleared" in out
    assert [c[0] for c in model.calls] == [[[1, 2]], [[3]]]          # nothing after /exit
    assert out.count("tokens per second") == 1                       # the table only while stats are on
    assert model.cleared == 1 and model.unloaded == 1


def test_shell_runs_commands_and_survives_failures(model, capsys, tmp_path):
    folder = str(tmp_path / "written")
    lines = ["models", "bogus command", "run", 'run m --sample-len 2 "7 8 9"', f"random {folder} --preset tiny_a --seed 3 --dtype float32",
             "random nowhere --preset no_such_preset", "", "exit", "models"]
    assert cli.cmd_shell(None, io.StringIO("\n".join(lines) + "\n")) == 0
    cap = capsys.readouterr()
    assert cap.out.count("(b200) burnlm> ") == len(lines) - 1        # a prompt for every line read, none after exit
    assert cap.out.count("| LlamaForCausalLM |") == 1
    assert "8 9" in cap.out and f"wrote {folder}" in cap.out
    assert "no preset named" in cap.err                              # the failing command was reported, the shell went on
    assert model.calls[0][0] == [[7, 8, 9]] and model.calls[0][1]["sample_len"] == 2
    cfg = json.load(open(os.path.join(folder, "config.json")))
    assert cfg["hidden_size"] == 64 and os.path.exists(os.path.join(folder, "model.safetensors"))


def test_the_default_command_is_the_shell(model, monkeypatch, capsys):
    monkeypatch.setattr("sys.stdin", io.StringIO("models\nquit\n"))
    assert cli.main([]) == 0
    assert "| LlamaForCausalLM |" in capsys.readouterr().out
