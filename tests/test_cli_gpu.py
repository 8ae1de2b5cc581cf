"""The command line end to end, as a user runs it: a model folder written by
``random-model``, tokens printed by ``generate``, and the same tokens from the Python
entry point on the same prompts (the reference drives its engine the same way from
tests/local_check.py:61-84)."""

import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_cli(*args):
    done = subprocess.run([sys.executable, "-m", "thing_htn_2026_b200", *args], cwd=ROOT, capture_output=True, text=True,
                          timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    return done.stdout.strip().splitlines()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_model_then_generate_prints_the_entry_points_tokens(tmp_path, dtype):
    from thing_htn_2026_b200 import Engine, cli
    folder = str(tmp_path / "model")
    assert run_cli("random-model", "--random-config", "tiny-b", "--seed", "1", "--out", folder, "--dtype", dtype,
                   "--gain-std", "0.1") == [folder]
    printed = [json.loads(line) for line in run_cli("generate", "--model", folder, "--shapes", "2x17x6,1x5x4",
                                                    "--seed", "0", "--dtype", dtype)]
    engine = Engine(folder, dtype=dtype)
    want = []
    for i, (b, s, n) in enumerate([(2, 17, 6), (1, 5, 4)]):
        steps = list(engine.generate(cli.make_prompt(b, s, engine.model.vocab_size, i), n))
        want += [[step[j] for step in steps] for j in range(b)]
    assert [p["tokens"] for p in printed] == want
    assert all(p["finish_reason"] == "length" for p in printed)

    # one batch of unequal prompts, sampled: --prompt-lens, --max-new-tokens, --temperature
    printed = [json.loads(line) for line in run_cli("generate", "--model", folder, "--prompt-lens", "1,23", "--seed", "7",
                                                    "--max-new-tokens", "12", "--temperature", "0.7", "--dtype", dtype)]
    prompts = cli.make_prompts_of([1, 23], engine.model.vocab_size, 7)
    steps = list(engine.generate(prompts, 12, temperature=0.7, seed=7))
    assert [p["tokens"] for p in printed] == [[step[j] for step in steps] for j in range(2)]


def test_generate_and_bench_from_a_named_configuration():
    printed = [json.loads(line) for line in run_cli("generate", "--random-config", "tiny-a", "--seed", "3",
                                                    "--prompt-lens", "5,9,16", "--max-new-tokens", "8")]
    assert len(printed) == 3 and all(len(p["tokens"]) == 8 for p in printed)
    lines = [json.loads(line) for line in run_cli("bench", "--random-config", "tiny-b", "--shapes", "2x16x8,1x40x5",
                                                  "--repeats", "1")]
    assert [line["shape"] for line in lines] == ["2x16x8", "1x40x5"]
    assert all(line["tok_per_s"] > 0 and line["ttft_ms"] > 0 for line in lines)


def test_the_other_architecture_from_the_command_line(tmp_path):
    """The same sub-commands on a Lanilix configuration: a folder written by ``random-model``
    is read back by ``generate``, chosen by the ``architecture`` key of its config.json, and
    prints the entry point's tokens."""
    from thing_htn_2026_b200 import Engine, cli
    folder = str(tmp_path / "lanilix")
    assert run_cli("random-model", "--random-config", "lanilix-tiny", "--seed", "2", "--out", folder, "--dtype",
                   "bfloat16") == [folder]
    with open(os.path.join(folder, "config.json")) as handle:
        assert json.load(handle)["architecture"] == "Lanilix"
    printed = [json.loads(line) for line in run_cli("generate", "--model", folder, "--prompt-lens", "3,70,21", "--seed", "5",
                                                    "--max-new-tokens", "9", "--dtype", "float32")]
    engine = Engine(folder, dtype="float32")
    steps = list(engine.generate(cli.make_prompts_of([3, 70, 21], engine.model.vocab_size, 5), 9))
    assert [p["tokens"] for p in printed] == [[step[j] for step in steps] for j in range(3)]
    lines = [json.loads(line) for line in run_cli("bench", "--random-config", "lanilix-tiny", "--layers", "2", "--shapes",
                                                  "2x16x8", "--repeats", "1")]
    assert lines[0]["shape"] == "2x16x8" and lines[0]["tok_per_s"] > 0


def test_a_bunudra_model_written_and_run_from_the_command_line(tmp_path):
    """The same for the third architecture: a named configuration written as a folder, read back by
    ``generate`` (chosen by the ``architecture`` key), the entry point's tokens, and ``bench``."""
    from thing_htn_2026_b200 import Engine, cli
    folder = str(tmp_path / "bunudra")
    assert run_cli("random-model", "--random-config", "bunudra-tiny", "--seed", "3", "--out", folder, "--dtype",
                   "bfloat16") == [folder]
    with open(os.path.join(folder, "config.json")) as handle:
        assert json.load(handle)["architecture"] == "Bunudra"
    printed = [json.loads(line) for line in run_cli("generate", "--model", folder, "--prompt-lens", "3,70,21", "--seed", "5",
                                                    "--max-new-tokens", "9", "--dtype", "float32")]
    engine = Engine(folder, dtype="float32")
    steps = list(engine.generate(cli.make_prompts_of([3, 70, 21], engine.model.vocab_size, 5), 9))
    assert [p["tokens"] for p in printed] == [[step[j] for step in steps] for j in range(3)]
    lines = [json.loads(line) for line in run_cli("bench", "--random-config", "bunudra-tiny", "--layers", "3", "--shapes",
                                                  "2x16x8", "--repeats", "1")]
    assert lines[0]["shape"] == "2x16x8" and lines[0]["tok_per_s"] > 0


def test_a_ditilix_model_written_and_run_from_the_command_line(tmp_path):
    """The same for the fourth architecture, with a layer that reads the layer before it: a named
    configuration written as a folder, read back by ``generate``, the entry point's tokens,
    ``bench``, and the replay program on the folder."""
    from thing_htn_2026_b200 import Engine, cli
    folder = str(tmp_path / "ditilix")
    assert run_cli("random-model", "--random-config", "ditilix-tiny", "--seed", "4", "--out", folder, "--dtype",
                   "bfloat16") == [folder]
    with open(os.path.join(folder, "config.json")) as handle:
        assert json.load(handle)["architecture"] == "Ditilix"
    printed = [json.loads(line) for line in run_cli("generate", "--model", folder, "--prompt-lens", "3,70,21", "--seed", "5",
                                                    "--max-new-tokens", "9", "--dtype", "float32")]
    engine = Engine(folder, dtype="float32")
    steps = list(engine.generate(cli.make_prompts_of([3, 70, 21], engine.model.vocab_size, 5), 9))
    assert [p["tokens"] for p in printed] == [[step[j] for step in steps] for j in range(3)]
    lines = [json.loads(line) for line in run_cli("bench", "--random-config", "ditilix-tiny", "--shapes", "2x16x8",
                                                  "--repeats", "1")]
    assert lines[0]["shape"] == "2x16x8" and lines[0]["tok_per_s"] > 0


def test_a_dubazen_model_written_and_run_from_the_command_line(tmp_path):
    """The same for the fifth architecture, with two copies of the stream, a scan, a pair of mixers and
    a layer without a feed-forward: a named configuration written as a folder, read back by
    ``generate``, the entry point's tokens, ``bench``, and the replay program on the folder."""
    from thing_htn_2026_b200 import Engine, cli
    folder = str(tmp_path / "dubazen")
    assert run_cli("random-model", "--random-config", "dubazen-tiny", "--seed", "4", "--out", folder, "--dtype",
                   "bfloat16") == [folder]
    with open(os.path.join(folder, "config.json")) as handle:
        assert json.load(handle)["architecture"] == "Dubazen"
    printed = [json.loads(line) for line in run_cli("generate", "--model", folder, "--prompt-lens", "3,70,21", "--seed", "5",
                                                    "--max-new-tokens", "9", "--dtype", "float32")]
    engine = Engine(folder, dtype="float32")
    steps = list(engine.generate(cli.make_prompts_of([3, 70, 21], engine.model.vocab_size, 5), 9))
    assert [p["tokens"] for p in printed] == [[step[j] for step in steps] for j in range(3)]
    lines = [json.loads(line) for line in run_cli("bench", "--random-config", "dubazen-tiny", "--shapes", "2x16x8",
                                                  "--repeats", "1")]
    assert lines[0]["shape"] == "2x16x8" and lines[0]["tok_per_s"] > 0
