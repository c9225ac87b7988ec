import pytest

from rosellm_b200 import cli_generate as C


def test_parse_rules():
    a = C.parse_args(["--model", "m", "--prompt", "hi"])
    assert (a.max_new_tokens, a.top_k, a.top_p, a.temperature, a.stop_on_eos, a.do_sample) == (100, 0, 1.0, 1.0, True, False)
    assert C.parse_args(["--checkpoint-path", "m", "--prompt", "x"]).model == "m"
    assert C.parse_args(["--hf-model-id", "m", "--prompt", "x", "--no-stop-on-eos"]).stop_on_eos is False
    assert C.parse_args(["--model", "m", "--interactive"]).prompt is None
    assert C.parse_args(["--random-weights", "c.json", "--prompt-ids", "1,2"]).prompt_ids == "1,2"
    with pytest.raises(SystemExit):
        C.parse_args(["--prompt", "x"])
    with pytest.raises(SystemExit):
        C.parse_args(["--model", "m"])


def test_chat_prompt_template():
    text = C.build_chat_prompt("be brief", [("hi", "hello\nthere")], "two\nlines")
    assert text.split("\n") == ["System:", "  be brief", "User:", "  hi", "Assistant:", "  hello", "  there",
                                "User:", "  two", "  lines", "Assistant:", "  "]
    assert C.build_chat_prompt("", [], "q").split("\n") == ["User:", "  q", "Assistant:", "  "]
    assert C.clean_reply("  sure\nmore\nUser:\n  next") == "sure\nmore"
    assert C.clean_reply("Assistant: ok\nSystem: x") == "ok"


class FakeEngine:
    def __init__(self):
        self.prompts = []

    def generate(self, prompt, **kw):
        self.prompts.append((prompt, kw))
        return f"reply {len(self.prompts)}\nUser:\n  ignored"


def test_interactive_loop_with_a_fake_engine():
    eng = FakeEngine()
    args = C.parse_args(["--model", "m", "--interactive", "--prompt", "first", "--system-prompt", "sys",
                         "--max-new-tokens", "7", "--do-sample", "--temperature", "0.5"])
    said = iter(["", "second", "/clear", "third", "/quit", "never"])
    out = []
    C.run_interactive(eng, args, read=lambda _: next(said), write=out.append)
    assert [p.split("\n")[-3] for p, _ in eng.prompts] == ["  first", "  second", "  third"]
    assert "reply 1" in eng.prompts[1][0] and "reply 2" not in eng.prompts[2][0]  # /clear forgot the history
    assert eng.prompts[0][1]["max_new_tokens"] == 7 and eng.prompts[0][1]["do_sample"] is True
    assert "Assistant> reply 3" in out and out[-1].endswith("exiting interactive mode.")
