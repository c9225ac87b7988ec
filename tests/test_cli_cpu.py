import pytest

from rosellm_b200 import cli_generate as C


def test_parse_rules():
    a = C.parse_args(["--model", "m", "--prompt", "hi"])
    assert (a.max_new_tokens, a.top_k, a.top_p, a.temperature, a.stop_on_eos, a.do_sample) == (100, 0, 1.0, 1.0, True, False)
    assert C.parse_args(["--checkpoint-path", "m", "--prompt", "x"]).model == "m"
    assert C.parse_args(["--hf-model-id", "m", "--prompt", "x", "--no-stop-on-eos"]).stop_on_eos is False
    assert C.parse_args(["--model", "m", "--interactive"]).prompt is None
    assert C.parse_args(["--random-weights", "c.json", "--prompt-ids", "1,2"]).prompt_ids == "1,2"
    a = C.parse_args(["--model", "m", "--prompt", "x", "--dtype", "fp32", "--num-pages", "9", "--max-num-batched-tokens",
                      "256", "--max-batch-size", "3", "--gpu-memory-utilization", "0.5"])
    assert (a.dtype, a.num_pages, a.max_num_batched_tokens, a.max_num_seqs, a.gpu_memory_utilization) == \
        ("fp32", 9, 256, 3, 0.5)
    assert C.parse_args(["--model", "m", "--prompt", "x", "--max-num-seqs", "5"]).max_num_seqs == 5
    with pytest.raises(SystemExit):
        C.parse_args(["--model", "m", "--prompt", "x", "--no-amp", "--dtype", "bf16"])
    with pytest.raises(SystemExit):
        C.parse_args(["--model", "m", "--prompt-ids", "1", "--prompt-ids-file", "f"])
    with pytest.raises(SystemExit):
        C.parse_args(["--prompt", "x"])
    with pytest.raises(SystemExit):
        C.parse_args(["--model", "m"])


def test_prompt_ids_from_a_file(tmp_path):
    f = tmp_path / "ids.txt"
    f.write_text("5, 17,3\n 9\t11\n")
    a = C.parse_args(["--model", "m", "--prompt-ids-file", str(f)])
    assert C.prompt_ids_of(a) == [5, 17, 3, 9, 11]
    assert C.prompt_ids_of(C.parse_args(["--model", "m", "--prompt-ids", "1,2, 3"])) == [1, 2, 3]
    assert C.prompt_ids_of(C.parse_args(["--model", "m", "--prompt", "text"])) is None


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


def test_the_status_word_is_read_by_every_way_of_running_the_engine():
    """``step`` (when the engine runs dry) and ``stream_generate`` read the kernels' status
    word, not only ``generate``: a fake runner whose word is set makes both raise."""
    from rosellm_b200.engine.llm import InferenceEngine
    from rosellm_b200.ops.kernels import KernelError

    class Runner:
        checks = 0

        def check_status(self):
            Runner.checks += 1
            raise KernelError("a kernel refused part of its input: a token id outside the embedding table")

    class Sched:
        def has_unfinished(self):
            return False

    eng = object.__new__(InferenceEngine)
    eng.runner, eng.scheduler, eng.overlap_schedule = Runner(), Sched(), True
    eng._inflight, eng._since_status_check, eng._requests, eng._finished_ids = None, 0, {}, []
    with pytest.raises(KernelError, match="token id"):
        eng.step()
    assert Runner.checks == 1

    # stream_generate: one request that a (fake) step finishes at once
    eng.add_request = lambda *a, **k: 0
    state = {"left": 1}
    eng.has_unfinished = lambda: state["left"] > 0

    def one_step():
        state["left"] -= 1
        return {0: 42}
    eng._step = one_step
    with pytest.raises(KernelError):
        list(eng.stream_generate([1, 2, 3], max_new_tokens=1))
    assert Runner.checks == 2
