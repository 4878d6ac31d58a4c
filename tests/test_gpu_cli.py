"""The command line as a user runs it (crates/engine/examples/generate.rs:15-71,
crates/engine/examples/load_weights.rs:11-28): `random_weights` writes a model folder,
`load_weights` counts its parameters, `bin/generate` prints the tokens the plain implementation
picks; with a tokenizer.json in the folder a text prompt goes in and text comes out; with
--random-weights the folder needs only its config.json."""
import json
import os
import re
import subprocess
import sys

import pytest

from tests.plain import llama_plain as plain
from tests.util import TINY_A

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args, timeout=900):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    return subprocess.run(list(args), capture_output=True, text=True, timeout=timeout, cwd=ROOT, env=env)


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    """A model folder made by the `random_weights` command from a config.json: tiny A with a
    vocabulary of 320 (so that the 300-word tokenizer's ids fit) and eos = the tokenizer's EOS."""
    from tests.test_tokenizer import make_tokenizer_json
    base = tmp_path_factory.mktemp("cli")
    d = TINY_A.to_dict()
    d.update(vocab_size=320, eos_token_id=1, bos_token_id=0)
    cfg_path = base / "config_in.json"
    cfg_path.write_text(json.dumps(d))
    model_dir = str(base / "model")
    p = run(sys.executable, "-m", "vllm_oxide_b200", "random_weights", model_dir, "--config", str(cfg_path), "--seed", "11",
            "--std", "0.08", "--dtype", "float32")
    assert p.returncode == 0, p.stderr[-2000:]
    assert os.path.exists(os.path.join(model_dir, "model.safetensors")) and os.path.exists(os.path.join(model_dir, "config.json"))
    make_tokenizer_json(model_dir)
    return model_dir


def test_load_weights_command_counts_the_parameters(folder):
    p = run(sys.executable, "-m", "vllm_oxide_b200", "load_weights", folder)
    assert p.returncode == 0, p.stderr[-2000:]
    m = re.search(r"params=(\d+) expected=(\d+)", p.stdout)
    cfg, tensors = plain.load_model(folder)
    assert m and int(m.group(1)) == int(m.group(2)) == sum(t.numel() for t in tensors.values())


def test_generate_command_prints_the_plain_tokens(folder):
    prompt = [5, 17, 3, 200, 41, 9, 77]
    p = run(os.path.join(ROOT, "bin", "generate"), folder, "--prompt-ids", ",".join(map(str, prompt)), "--max-new", "8",
            "--dtype", "float32")
    assert p.returncode == 0, p.stderr[-2000:]
    cfg, tensors = plain.load_model(folder)
    want = plain.greedy_generate(cfg, tensors, prompt, 8, stop=1)
    # with a tokenizer in the folder the output is text: the words of the picked tokens
    from vllm_oxide_b200.engine.tokenizer import TextTokenizer
    tok = TextTokenizer.load(folder)
    assert p.stdout.strip() == tok.decode(want)
    stats = json.loads([l for l in p.stderr.splitlines() if l.startswith("{")][-1])
    assert stats["prompt_tokens"] == len(prompt) and stats["generated"] == len(want)
    assert stats["prefill_tok_s"] > 0 and stats["workspace_high_water_mb"] > 0


def test_generate_command_takes_a_text_prompt(folder):
    """Positional arguments as the reference's example: model folder, prompt, max_new."""
    from vllm_oxide_b200.engine.tokenizer import TextTokenizer
    tok = TextTokenizer.load(folder)
    text = "w5 w17 w100 w250"
    p = run(sys.executable, "-m", "vllm_oxide_b200", "generate", folder, text, "6", "--dtype", "float32", "--no-cuda-graphs")
    assert p.returncode == 0, p.stderr[-2000:]
    ids = tok.encode(text)
    assert ids[0] == 0 and len(ids) == 5                       # BOS first
    cfg, tensors = plain.load_model(folder)
    want = plain.greedy_generate(cfg, tensors, ids, 6, stop=1)
    assert p.stdout.strip() == tok.decode(want)


def test_generate_command_with_random_weights_needs_only_config_json(folder, tmp_path):
    """--random-weights SEED: the same tokens as the Python entry point with the same seed."""
    bare = tmp_path / "bare"
    bare.mkdir()
    (bare / "config.json").write_text(open(os.path.join(folder, "config.json")).read())
    prompt = [9, 8, 7, 300, 6]
    p = run(os.path.join(ROOT, "bin", "generate"), str(bare), "--prompt-ids", ",".join(map(str, prompt)), "--max-new", "7",
            "--dtype", "float32", "--random-weights", "5", "--random-weights-std", "0.3")
    assert p.returncode == 0, p.stderr[-2000:]
    got = [int(t) for t in p.stdout.split()]
    from vllm_oxide_b200.engine import LLM
    from vllm_oxide_b200.sampling import SamplingParams
    llm = LLM(str(bare), dtype="float32", random_weights_seed=5, random_weights_std=0.3, max_batch_tokens=64, max_seqs=2, max_model_len=64, num_pages=16)
    want = llm.generate([prompt], SamplingParams(max_new_tokens=7))[0].token_ids
    assert got == want and 1 <= len(got) <= 7
    other = LLM(str(bare), dtype="float32", random_weights_seed=6, random_weights_std=0.3, max_batch_tokens=64, max_seqs=2, max_model_len=64, num_pages=16)
    assert other.generate([prompt], SamplingParams(max_new_tokens=7))[0].token_ids != want


def test_unknown_command_and_bad_folder():
    p = run(sys.executable, "-m", "vllm_oxide_b200", "nosuch")
    assert p.returncode == 2
    p = run(os.path.join(ROOT, "bin", "generate"), "/nonexistent/model", "--prompt-ids", "1,2")
    assert p.returncode != 0 and "config.json" in (p.stderr + p.stdout)
