"""Another architecture without a change to the framework's files.

``tests/toy_arch.py`` registers a mixer with state of its own, a feed-forward with routing, a
position encoding with a tensor of its own and the architecture ``ToyForCausalLM`` through the
public hooks. Here it goes the whole way a user's model goes: registry, a model folder written by
the random-weights mode, the loader, ``Engine.generate`` with the default options, the command
line with ``--plugin``, trace replay; and its tokens and logits must be those of a plain numpy
restatement. The reference dispatches on the checkpoint's architecture string in the same place
(garuda/src/server/mod.rs:372-377) and chooses the feed-forward and the per-layer cache needs from
the checkpoint (garuda/src/llama/mod.rs:495-507, garuda/src/cache/mod.rs:163-171, :630-648).

Also here: the branches of the built-in parts that the Llama model never takes (no position
encoding, an encoding applied outside the fused kernel, a rotation narrower than the head).
The first tests run on the CPU stand-in for the kernels; the ``gpu`` ones on the device.
"""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from tests import toy_arch
from tests.helpers import ROOT, TraceRunner, assert_close, folder_weights
from tests.plain import llama_plain
from tests.plain.cpu_ops import CpuOps

CFG = toy_arch.TOY_CONFIG
_DIR = {}


def toy_dir():
    from garuda_b200.weights import write_random_model
    if "d" not in _DIR:
        _DIR["d"] = tempfile.mkdtemp(prefix="garuda_toy_")
        write_random_model(_DIR["d"], CFG, seed=3, store_dtype=torch.float32)
    return _DIR["d"]


def toy_tokens(n, seed):
    return np.random.default_rng(seed).integers(0, CFG["vocab_size"], n).tolist()


def plain(tokens):
    return toy_arch.plain_forward(CFG, folder_weights(toy_dir()), tokens)


def greedy(prompt, n):
    return toy_arch.plain_greedy(CFG, folder_weights(toy_dir()), prompt, n)


def step_through(engine, dtype):
    """Whole, then in portions down to one token beside a second request, against the plain model."""
    from garuda_b200 import StepEntry
    toks, other = toy_tokens(40, 0), toy_tokens(25, 1)
    ref, ref_other = plain(toks), plain(other)
    out = engine.step([StepEntry(1, toks, range(40))]).float().cpu().numpy()
    engine.runner.end(1)
    assert_close(out, ref, dtype, "toy: whole", config="toy")
    outs, outs_other, pos, pos_other = [], [], 0, 0
    for c, c_other in ((7, 3), (2, 1), (11, 9), (1, 1), (19, 11)):
        o = engine.step([StepEntry(2, toks[pos:pos + c], range(c)),
                         StepEntry(3, other[pos_other:pos_other + c_other], range(c_other))]).float().cpu().numpy()
        outs.append(o[:c].copy()), outs_other.append(o[c:].copy())
        pos, pos_other = pos + c, pos_other + c_other
    engine.runner.end(2), engine.runner.end(3)
    assert_close(np.concatenate(outs), ref, dtype, "toy: portions", config="toy")
    assert_close(np.concatenate(outs_other), ref_other, dtype, "toy: portions of the second request", config="toy")


def generate_with_reused_slots_and_preemption(make_engine):
    """More prompts than slots, so that every slot is taken again by a request that must not see
    its predecessor's running mean; then so few pages that a request is sent back and recomputed."""
    from garuda_b200 import SamplingParams
    prompts = [toy_tokens(n, 10 + i) for i, n in enumerate((5, 17, 9, 3, 12, 7))]
    want = [greedy(p, 8) for p in prompts]
    roomy = make_engine(max_concurrent=2)
    got = roomy.generate(prompts, SamplingParams.greedy(max_tokens=8))
    assert [r.tokens for r in got] == want and all(r.finish_reason == "length" for r in got)
    tight = make_engine(max_concurrent=3, kv_tokens=48, page_size=8)
    got = tight.generate(prompts, SamplingParams.greedy(max_tokens=8))
    assert tight.stats()["preemptions"] > 0
    assert [r.tokens for r in got] == want


# ---------------------------------------------------------------------- CPU
def test_toy_architecture_registry_folder_loader_and_steps_on_the_cpu_stand_in():
    from garuda_b200 import Engine, registered_architectures
    assert "ToyForCausalLM" in registered_architectures()
    e = Engine(toy_dir(), dtype="float32", page_size=8, ops=CpuOps(), max_concurrent=4)
    assert not e.model.graph_safe            # the toy parts say nothing, so nothing of it is captured
    assert len(e.model.state_calls) == 1 and len(e.model.cache_groups) == 2      # windowed and not
    step_through(e, "float32")


def test_toy_generation_with_reused_slots_and_preemption_on_the_cpu_stand_in():
    from garuda_b200 import Engine
    generate_with_reused_slots_and_preemption(
        lambda **kw: Engine(toy_dir(), dtype="float32", ops=CpuOps(), **{"page_size": 8, **kw}))


def test_a_folder_of_the_toy_architecture_is_checked_like_any_other():
    from garuda_b200 import Engine, WeightError
    from garuda_b200.weights import write_random_model
    from garuda_b200.weights.safetensors_io import SafetensorsFolder, write_safetensors
    d = tempfile.mkdtemp(prefix="garuda_toy_bad_")
    write_random_model(d, CFG, seed=3)
    f = SafetensorsFolder(d)
    tensors = {n: f.tensor(n) for n in f.names()}
    del tensors["blocks.0.attention.position.table"]
    tensors["blocks.1.mean.gain"] = tensors["blocks.1.mean.gain"][:-1].contiguous()
    tensors["lm_head.weight"] = tensors["out.weight"]          # this architecture ignores no name
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightError) as err:
        Engine(d, dtype="float32", ops=CpuOps())
    assert err.value.missing == ["blocks.0.attention.position.table"]
    assert err.value.unexpected == ["lm_head.weight"]
    assert [w[0] for w in err.value.wrong_shape] == ["blocks.1.mean.gain"]


def _attention_alone(ops, dtype, position, T=23, window=None):
    """The attention part alone in two steps; returns (output, its tensors as float32 numpy, inputs)."""
    from garuda_b200.parts import PagedAttention, LayerCache
    from garuda_b200.engine.batch import StepBatch, StepContext, Workspace
    dev = getattr(ops, "device", "cpu")
    d, Hq, Hkv, hd, page = 48, 4, 2, 16, 8
    att = PagedAttention(d, Hq, Hkv, hd, position=position, window=window)
    g = torch.Generator().manual_seed(5)
    ws = {k: (torch.randn(v.shape, generator=g) * (0.3 if "proj" in k else 1.0)).to(dtype if "proj" in k else torch.float32)
          for k, v in att.tensors().items()}
    att.load({k: v.to(dev) for k, v in ws.items()}, ops, dtype)
    h = torch.randn(T, d, generator=g).to(dtype)
    k_pool = torch.zeros(6, Hkv, page, hd, dtype=dtype, device=dev)
    v_pool = torch.zeros_like(k_pool)
    bt = torch.tensor([[4, 1, 3, 0]], dtype=torch.int32, device=dev)
    outs = []
    for start, n in ((0, 14), (14, T - 14)):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        batch = StepBatch(num_tokens=n, num_requests=1, token_ids=i32([0] * n), positions=i32(list(range(start, start + n))),
                          token_req=i32([0] * n), cu_q=i32([0, n]), kv_lens=i32([start + n]), slots=i32([0]),
                          block_tables=[bt], logit_rows=i32([]), num_logit_rows=0, max_q_len=n, max_kv_len=start + n)
        ctx = StepContext(batch=batch, ws=Workspace(dev), ops=ops, dtype=dtype)
        cache = LayerCache(need=att.cache_need(), k=k_pool, v=v_pool, block_table=bt, page_size=page)
        outs.append(att.forward(ctx, h[start:start + n].to(dev), cache).float().cpu())
    return torch.cat(outs).numpy(), {k: v.float().numpy() for k, v in ws.items()}, h.float().numpy()


def _plain_attention(w, h, change, window=None, Hq=4, Hkv=2, hd=16):
    T = h.shape[0]
    q = llama_plain.linear(h, w["q_proj.weight"]).reshape(T, Hq, hd)
    k = llama_plain.linear(h, w["k_proj.weight"]).reshape(T, Hkv, hd)
    v = llama_plain.linear(h, w["v_proj.weight"]).reshape(T, Hkv, hd)
    q, k = change(q), change(k)
    return llama_plain.linear(llama_plain.attention(q, k, v, window), w["o_proj.weight"])


POSITIONS = {
    "none": ({"name": "none", "params": {}}, lambda w, pos: (lambda t: t)),
    "learned": ({"name": "toy_learned", "params": {"positions": 64, "head_dim": 16}},
                lambda w, pos: (lambda t: t + w["position.table"][pos][:, None, :])),
    # the first 8 channels of every head only, pairs (i, i + 4): narrower than the fused kernel's pairs
    "narrow": ({"name": "rotary", "params": {"theta": 100.0, "head_dim": 16, "layout": "half", "rotary_dim": 8}},
               lambda w, pos: (lambda t: np.concatenate(
                   [llama_plain.rope(t[..., :8], pos, 100.0, "half"), t[..., 8:]], axis=-1))),
    # the same width with pairs (2i, 2i + 1): runs in the fused kernel, the other pairs at frequency zero
    "narrow-interleaved": ({"name": "rotary", "params": {"theta": 100.0, "head_dim": 16, "layout": "interleaved",
                                                         "rotary_dim": 8}},
                           lambda w, pos: (lambda t: np.concatenate(
                               [llama_plain.rope(t[..., :8], pos, 100.0, "interleaved"), t[..., 8:]], axis=-1))),
}


@pytest.mark.parametrize("kind", sorted(POSITIONS))
def test_position_encodings_the_llama_model_never_uses_on_the_cpu_stand_in(kind):
    position, change = POSITIONS[kind]
    got, w, h = _attention_alone(CpuOps(), torch.float32, position, window=9)
    ref = _plain_attention(w, h, change(w, np.arange(h.shape[0])), window=9)
    assert np.abs(got - ref).max() <= 2e-5 * np.abs(ref).max()


# ---------------------------------------------------------------------- GPU
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", sorted(POSITIONS))
def test_position_encodings_the_llama_model_never_uses(kind, dtype):
    from garuda_b200.kernels import CudaOps
    position, change = POSITIONS[kind]
    ops = CudaOps("cuda:0", tensor_cores=dtype == torch.bfloat16)
    got, w, h = _attention_alone(ops, dtype, position, window=9)
    ref = _plain_attention(w, h, change(w, np.arange(h.shape[0])), window=9)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(got - ref).max() <= tol * np.abs(ref).max()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_steps_on_the_gpu_with_default_options(dtype):
    """``Engine(...)`` as a user calls it: CUDA graphs are on by default, and the toy's decode steps
    are simply not captured, because its parts do not say that they may be."""
    from garuda_b200 import Engine
    e = Engine(toy_dir(), dtype=dtype, page_size=8)
    assert e.runner.graphs is not None and not e.model.graph_safe
    step_through(e, dtype)
    assert e.runner.graphs.replays == 0
    e.check_errors()


@pytest.mark.gpu
def test_toy_generation_with_reused_slots_and_preemption():
    from garuda_b200 import Engine
    generate_with_reused_slots_and_preemption(
        lambda **kw: Engine(toy_dir(), dtype="float32", **{"page_size": 8, **kw}))


@pytest.mark.gpu
def test_toy_architecture_through_the_command_line_and_trace_replay(tmp_path):
    d = toy_dir()
    cfg = tmp_path / "config.toml"
    cfg.write_text(f'[model]\npath = "{d}"\ndtype = "float32"\ncontext = 96\nplugins = ["tests.toy_arch"]\n'
                   '[memory]\npage_size = 8\n[sampling]\ntemperature = 0.0\nmax_tokens = 7\n')
    prompt = toy_tokens(11, 42)
    garuda = [sys.executable, os.path.join(ROOT, "bin", "garuda")]
    out = subprocess.run(garuda + ["--config", str(cfg), "generate", "--prompt-ids", ",".join(map(str, prompt))],
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["tokens"] == greedy(prompt, 7) and rec["finish_reason"] == "length"
    # without the plugin the name is unknown, and the message says what is registered
    bare = tmp_path / "bare.toml"
    bare.write_text(f'[model]\npath = "{d}"\ndtype = "float32"\n')
    out = subprocess.run(garuda + ["--config", str(bare), "inspect", d], capture_output=True, text=True)
    assert out.returncode == 1 and "ToyForCausalLM" in out.stdout and "LlamaForCausalLM" in out.stdout
    out = subprocess.run(garuda + ["--plugin", "tests.toy_arch", "--config", str(bare), "inspect", d],
                         capture_output=True, text=True)
    assert out.returncode == 0 and "loadable: yes" in out.stdout, out.stdout + out.stderr
    # `garuda replay` on a trace file, and bin/trace_run with --plugin, give the plain model's logits
    toks = toy_tokens(30, 8)
    trace = tmp_path / "trace.jsonl"
    trace.write_text("\n".join(json.dumps(s) for s in (
        {"step": 0, "entries": [{"id": "a", "tokens": toks[:19], "want": [0, 18]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": toks[19:21], "want": [1]}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": toks[21:], "want": list(range(9))}], "end": ["a"]})) + "\n")
    outdir = tmp_path / "logits"
    out = subprocess.run(garuda + ["--config", str(cfg), "replay", str(trace), str(outdir)], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert out.stdout.split() == ["done", "0", "done", "1", "done", "2"]
    got = np.concatenate([np.fromfile(outdir / f"{i}.f32", dtype="<f4").reshape(-1, CFG["vocab_size"]) for i in range(3)])
    ref = plain(toks)
    assert_close(got, ref[[0, 18, 20] + list(range(21, 30))], "float32", "toy: garuda replay", config="toy")
    tr = TraceRunner(d, "float32", max_tokens=128, extra=["--plugin", "tests.toy_arch", "--page-size", "8"])
    got = tr.step([("x", toks, range(30))], end=["x"])
    assert tr.close() == 0
    assert_close(got, ref, "float32", "toy: bin/trace_run", config="toy")


@pytest.mark.gpu
def test_a_wait_that_runs_out_ends_the_step_with_an_error_and_the_engine_goes_on():
    """A kernel whose bounded wait runs out records a code and returns; the host sees it where it
    waits for the step's tokens, the step's requests end with an error, and the next requests run.
    The wait here is one that nothing ever completes (a barrier without arrivals, limit one
    millisecond), launched between a step and the collection of its tokens."""
    from garuda_b200 import Engine, SamplingParams
    from garuda_b200.kernels.ops import KernelError
    from tests.helpers import model_dir, random_tokens
    e = Engine(model_dir("A", torch.bfloat16), dtype="bfloat16", page_size=16, lookahead=False)
    prompt = random_tokens("A", 9, 1)
    good = e.generate([prompt], SamplingParams.greedy(max_tokens=5))[0]
    assert good.finish_reason == "length"
    # the status alone
    e.ops.tc.selftest_wait_runs_out(1000)
    torch.cuda.synchronize()
    assert e.ops.failed_wait() == 1
    with pytest.raises(KernelError, match="never arrived"):
        e.check_errors()
    assert e.ops.failed_wait() == 0
    e.check_errors()
    # inside a generation: the third step's kernels are followed by the wait that runs out
    steps = {"n": 0}
    run = e.runner.run

    def run_then_fail(entries, device_tokens=None):
        out = run(entries, device_tokens)
        steps["n"] += 1
        if steps["n"] == 3:
            e.ops.tc.selftest_wait_runs_out(1000)
        return out

    e.runner.run = run_then_fail
    bad = e.generate([prompt], SamplingParams.greedy(max_tokens=5))[0]
    e.runner.run = run
    assert bad.finish_reason == "error" and "gave up waiting" in bad.error and len(bad.tokens) == 2
    st = e.stats()
    assert st["failed"] == 1 and st["pages_free"] == st["pages_total"]
    again = e.generate([prompt], SamplingParams.greedy(max_tokens=5))[0]
    assert again.tokens == good.tokens and again.finish_reason == "length"
