"""The command line's parts that need no GPU: `init` (random-weights mode), `inspect` (what a
folder holds and whether it will load: garuda/src/main.rs:56-148), the configuration file before
the subcommand with defaults when it does not exist (garuda/src/cli/mod.rs:10-44,
garuda/src/main.rs:30-36), and what is refused."""
import json
import os

import pytest

from garuda_b200.cli import main
from tests.helpers import TINY_A, TINY_B


def run(capsys, *argv):
    rc = main(list(argv))
    out = capsys.readouterr()
    return rc, out.out, out.err


def test_init_writes_a_folder_that_inspect_says_will_load(tmp_path, capsys):
    cj = tmp_path / "cfg.json"
    cj.write_text(json.dumps(TINY_B))
    folder = tmp_path / "model"
    rc, out, _ = run(capsys, "init", str(folder), "--config-json", str(cj), "--seed", "7", "--store-dtype", "float32")
    assert rc == 0 and "seed 7" in out
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    assert json.loads((folder / "config.json").read_text())["hidden_size"] == TINY_B["hidden_size"]
    rc, out, _ = run(capsys, "-c", str(tmp_path / "absent.toml"), "inspect", str(folder))
    assert rc == 0 and "loadable: yes" in out and "architecture: LlamaForCausalLM" in out
    assert "rope_theta = 500000.0" in out and "model.layers.2.mlp.down_proj.weight" in out
    assert "lm_head.weight" not in out                        # tied: the head is the embedding table
    # the same seed gives the same bytes, another seed other bytes
    again = tmp_path / "again"
    other = tmp_path / "other"
    run(capsys, "init", str(again), "--config-json", str(cj), "--seed", "7", "--store-dtype", "float32")
    run(capsys, "init", str(other), "--config-json", str(cj), "--seed", "8", "--store-dtype", "float32")
    same = (folder / "model.safetensors").read_bytes() == (again / "model.safetensors").read_bytes()
    differs = (folder / "model.safetensors").read_bytes() != (other / "model.safetensors").read_bytes()
    assert same and differs


def test_inspect_names_what_is_wrong_with_a_folder(tmp_path, capsys):
    from garuda_b200.weights import write_random_model
    from garuda_b200.weights.safetensors_io import SafetensorsFolder, write_safetensors
    import torch
    folder = tmp_path / "m"
    write_random_model(str(folder), TINY_A, 0, store_dtype=torch.float32)
    f = SafetensorsFolder(str(folder))
    tensors = {n: f.tensor(n) for n in f.names()}
    del tensors["model.layers.1.self_attn.o_proj.weight"]
    tensors["model.layers.0.mlp.up_proj.weight"] = tensors["model.layers.0.mlp.up_proj.weight"][:-1].contiguous()
    tensors["extra.weight"] = torch.zeros(3)
    write_safetensors(str(folder / "model.safetensors"), tensors)
    rc, out, _ = run(capsys, "inspect", str(folder))
    assert rc == 1 and "loadable: no" in out
    assert "missing: model.layers.1.self_attn.o_proj.weight" in out
    assert "unexpected: extra.weight" in out and "wrong shape: model.layers.0.mlp.up_proj.weight" in out
    # a config.json the engine cannot honour
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text(json.dumps(dict(TINY_A, rope_scaling={"type": "linear", "factor": 2.0})))
    rc, out, _ = run(capsys, "inspect", str(bad))
    assert rc == 1 and "rope_scaling" in out and "loadable: no" in out
    # an architecture nobody registered
    (bad / "config.json").write_text(json.dumps(dict(TINY_A, architectures=["NobodyForCausalLM"])))
    rc, out, _ = run(capsys, "inspect", str(bad))
    assert rc == 1 and "NobodyForCausalLM" in out and "LlamaForCausalLM" in out


def test_what_the_command_line_refuses(tmp_path, capsys):
    rc, _, err = run(capsys, "serve")
    assert rc == 2 and "no server" in err
    rc, _, err = run(capsys)
    assert rc == 2 and "generate" in err
    cfg = tmp_path / "config.toml"
    cfg.write_text("[model]\nbogus = 1\n")
    rc, _, err = run(capsys, "-c", str(cfg), "generate", "--prompt-ids", "1,2")
    assert rc == 1 and "bogus" in err
    cfg.write_text("[server]\nrequest_timeout_secs = 0\n")
    rc, _, err = run(capsys, "-c", str(cfg), "benchmark")
    assert rc == 1 and "request_timeout_secs" in err
    with pytest.raises(SystemExit):                           # the subcommand's own options are checked by the parser
        main(["generate"])
    capsys.readouterr()
