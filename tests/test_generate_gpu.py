"""Generation through the Python entry point and the command line on the GPU,
each part of the model alone, and a toy mixer with state of its own that is
registered, built and stepped without a change to the framework's files."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests.helpers import (TINY, ROOT, model_dir, plain_logits, random_tokens, assert_close, folder_weights, TOL,
                           tolerance)
from tests.plain import llama_plain
from tests.plain.cpu_ops import CpuOps

pytestmark = pytest.mark.gpu
STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_float32(name):
    from garuda_b200 import Engine, SamplingParams
    cfg = TINY[name][0]
    e = Engine(model_dir(name), dtype="float32", page_size=16, max_concurrent=4, max_batch_tokens=48,
               prefill_chunk=20)
    prompts = [random_tokens(name, n, 50 + n) for n in (5, 41, 1, 63, 17, 30)]
    res = e.generate(prompts, SamplingParams.greedy(max_tokens=12))
    w = folder_weights(model_dir(name))
    for p, r in zip(prompts, res):
        assert r.finish_reason == "length" and r.tokens == llama_plain.greedy_generate(cfg, w, p, 12)
    st = e.stats()
    assert st["completed"] == 6 and st["pages_free"] == st["pages_total"]
    e.cache.manager.check_invariants()
    assert e.runner.graphs.replays > 0                     # decode steps came from captured graphs


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_bfloat16(name):
    """bfloat16 may turn a near-tie the other way; every generated token must be a
    near-maximum of the plain model's logits given the same prefix."""
    from garuda_b200 import Engine, SamplingParams
    cfg = TINY[name][0]
    e = Engine(model_dir(name, torch.bfloat16), dtype="bfloat16", page_size=16, max_concurrent=4)
    prompts = [random_tokens(name, n, 90 + n) for n in (9, 33, 2)]
    res = e.generate(prompts, SamplingParams.greedy(max_tokens=10))
    w = folder_weights(model_dir(name, torch.bfloat16))
    for p, r in zip(prompts, res):
        assert len(r.tokens) == 10
        logits = llama_plain.forward(cfg, w, list(p) + r.tokens)
        for i, tok in enumerate(r.tokens):
            row = logits[len(p) - 1 + i]
            # the engine's logit of the token it chose is its largest, and both that logit and the
            # plain model's are within the configuration's tolerance of each other
            assert row[tok] >= row.max() - 2 * tolerance("bfloat16", name) * np.abs(row).max()
    e.ops.tc.check_errors()


def test_sampled_generation_is_seeded_and_follows_the_plain_sampler():
    from garuda_b200 import Engine, SamplingParams
    from tests.plain.sampling_plain import Rng, sample as plain_sample
    cfg = TINY["A"][0]
    e = Engine(model_dir("A"), dtype="float32", page_size=16)
    prompt = random_tokens("A", 12, 3)
    params = SamplingParams(temperature=0.9, top_k=20, top_p=0.9, max_tokens=8, seed=1234)
    res = e.generate([prompt, prompt], [params, params])
    assert res[0].tokens == res[1].tokens
    w = folder_weights(model_dir("A"))
    rng, seq, want = Rng(1234), list(prompt), []
    for _ in range(8):
        tok = plain_sample(llama_plain.forward(cfg, w, seq)[-1], 0.9, 20, 0.9, rng)
        want.append(tok)
        seq.append(tok)
    assert res[0].tokens == want


def test_preemption_on_the_gpu_keeps_the_tokens():
    from garuda_b200 import Engine, SamplingParams
    prompts = [random_tokens("A", 20, 70 + i) for i in range(3)]
    roomy = Engine(model_dir("A"), dtype="float32", page_size=8, max_concurrent=3)
    want = roomy.generate(prompts, SamplingParams.greedy(max_tokens=24))
    tight = Engine(model_dir("A"), dtype="float32", page_size=8, kv_tokens=96, max_concurrent=3)
    got = tight.generate(prompts, SamplingParams.greedy(max_tokens=24))
    assert tight.stats()["preemptions"] > 0
    assert [r.tokens for r in got] == [r.tokens for r in want]


def test_graphs_captured_ahead_of_time_and_among_dropped_engines():
    """``warm_up`` captures every batch size's graph before any request; the tokens are those of an
    engine without graphs. Engines dropped in between leave garbage that holds graphs and device
    memory: a capture must not be invalidated by its collection."""
    import gc
    from garuda_b200 import Engine, SamplingParams
    name = "A"
    prompts = [random_tokens(name, n, 500 + n) for n in (3, 21, 9, 14)]
    params = [SamplingParams.greedy(max_tokens=m) for m in (12, 5, 9, 2)]
    kw = dict(dtype="bfloat16", page_size=16, max_concurrent=4)
    want = Engine(model_dir(name, torch.bfloat16), cuda_graphs=False, **kw).generate(prompts, params)
    for _ in range(3):
        e = Engine(model_dir(name, torch.bfloat16), **kw)
        gc.set_threshold(1)           # collect at every allocation: also in the middle of a capture
        try:
            e.warm_up()
        finally:
            gc.set_threshold(700, 10, 10)
        assert sorted(e.runner.graphs.graphs) == [1, 2, 4]
        got = e.generate(prompts, params)
        assert [r.tokens for r in got] == [r.tokens for r in want]
        assert e.runner.graphs.replays > 0
        e.cycle = e                   # garbage that only a collection frees


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_change_nothing(dtype):
    """Decode steps, greedy or sampled, are launched before the tokens of the step in front have
    reached the host. Requests that end at different times (their own limits, an end-of-sequence token in the
    middle), more prompts than may run at once, and too few pages: the tokens and the reasons for
    finishing are those of an engine that launches nothing ahead."""
    from garuda_b200 import Engine, SamplingParams
    name = "D"
    prompts = [random_tokens(name, n, 300 + i) for i, n in enumerate([5, 40, 17, 64, 9, 33, 2])]
    limits = [7, 30, 12, 25, 40, 3, 18]
    params = [SamplingParams.greedy(max_tokens=m) for m in limits]
    # sampled requests among the greedy ones: their draws come from the requests' own generators
    for i in (1, 3, 6):
        params[i] = SamplingParams(temperature=0.9, top_k=50, top_p=0.95, max_tokens=limits[i], seed=40 + i)
    kw = dict(dtype=dtype, page_size=16, max_concurrent=3)
    plain = Engine(model_dir(name), lookahead=False, **kw).generate(prompts, params)
    # a token that some request produces in the middle of its answer ends it there
    eos = plain[4].tokens[11]
    for extra in (dict(), dict(eos_token_id=eos), dict(kv_tokens=160)):
        want = Engine(model_dir(name), lookahead=False, **kw, **extra).generate(prompts, params)
        ahead = Engine(model_dir(name), lookahead=True, **kw, **extra)
        got = ahead.generate(prompts, params)
        assert [r.tokens for r in got] == [r.tokens for r in want], extra
        assert [r.finish_reason for r in got] == [r.finish_reason for r in want], extra
        if "kv_tokens" in extra:
            assert ahead.stats()["preemptions"] > 0
        if "eos_token_id" in extra:
            assert any(r.finish_reason != "length" for r in want)


def test_a_timeout_between_steps_launched_ahead():
    """A request whose time runs out while a step for it is already in flight (launched ahead)
    ends with the error, the other goes on to the tokens of a run without limits, and nothing
    stays behind in the cache."""
    from garuda_b200 import Engine, SamplingParams
    prompts = [random_tokens("A", 9, 1), random_tokens("A", 5, 2), random_tokens("A", 7, 3)]
    params = [SamplingParams.greedy(max_tokens=m) for m in (40, 6, 40)]
    e = Engine(model_dir("A"), dtype="bfloat16", page_size=16, max_concurrent=3)
    free = e.generate(prompts, params)
    e.scheduler.set_time(10.0)
    count = [0]

    def on_token(i, tok):
        count[0] += 1
        if count[0] == 30:                       # ten tokens each, the second request long finished
            e.scheduler.set_time(20.0)

    res = e.generate(prompts, params, on_token=on_token, timeout=5.0)
    assert [r.finish_reason for r in res] == ["error", "length", "error"]
    assert res[0].error == res[2].error == "timeout" and res[1].tokens == free[1].tokens
    for got, want in zip(res, free):
        assert 0 < len(got.tokens) <= len(want.tokens) and got.tokens == want.tokens[:len(got.tokens)]
    st = e.stats()
    assert st["timed_out"] == 2 and st["running"] == 0 and st["pages_free"] == st["pages_total"]
    e.scheduler.set_time(30.0)
    again = e.generate(prompts, params)          # the engine goes on as before
    assert [r.tokens for r in again] == [r.tokens for r in free]
    e.cache.manager.check_invariants()
    e.check_errors()


def test_missing_extension_fails_loudly(monkeypatch):
    from garuda_b200.csrc import build
    from garuda_b200.kernels import ops as ops_mod
    monkeypatch.setattr(build, "_LOADED", {})
    monkeypatch.setattr(ops_mod, "load_kernel_lib", lambda name: (_ for _ in ()).throw(
        build.BuildError("nvcc was not found")))
    with pytest.raises(build.BuildError):
        ops_mod.CudaOps("cuda:0")


def test_command_line_generate_and_inspect(tmp_path):
    d = model_dir("A")
    cfg = tmp_path / "config.toml"
    cfg.write_text(f'[model]\npath = "{d}"\ndtype = "float32"\ncontext = 128\n[memory]\npage_size = 16\n'
                   '[sampling]\ntemperature = 0.0\nmax_tokens = 6\n')
    prompt = random_tokens("A", 9, 77)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "garuda"), "--config", str(cfg), "generate",
                          "--prompt-ids", ",".join(map(str, prompt))], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["tokens"] == llama_plain.greedy_generate(TINY["A"][0], folder_weights(d), prompt, 6)
    assert rec["finish_reason"] == "length"
    ins = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "garuda"), "inspect", d],
                         capture_output=True, text=True)
    assert ins.returncode == 0 and "LlamaForCausalLM" in ins.stdout and "loadable: yes" in ins.stdout


# ---------------------------------------------------------------------- parts alone
def _ctx(ops, dtype, batch):
    from garuda_b200.engine.batch import StepContext, Workspace
    return StepContext(batch=batch, ws=Workspace("cuda:0"), ops=ops, dtype=dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_feed_forward_and_block_alone(dtype):
    from garuda_b200.kernels import CudaOps
    from garuda_b200.parts import RMSNorm, SwiGLU
    ops = CudaOps("cuda:0", tensor_cores=dtype == torch.bfloat16)
    tol = 3e-6 if dtype == torch.float32 else 1.5e-2
    d, inner, T = 72, 200, 13
    x = torch.randn(T, d)
    norm = RMSNorm(d, 1e-6)
    w = 1 + 0.1 * torch.randn(d)
    norm.load({"weight": w.cuda()}, ops, dtype)
    ctx = _ctx(ops, dtype, None)
    got = norm.forward(ctx, x.cuda()).float().cpu()
    ref = llama_plain.rmsnorm(x.numpy(), w.numpy(), 1e-6)
    assert np.abs(got.numpy() - ref).max() <= tol * np.abs(ref).max()
    ff = SwiGLU(d, inner)
    ws = {k: (torch.randn(v.shape) * 0.1).to(dtype) for k, v in ff.tensors().items()}
    ff.load({k: v.cuda() for k, v in ws.items()}, ops, dtype)
    h = (torch.randn(T, d)).to(dtype)
    res = torch.randn(T, d)
    acc = res.clone().cuda()
    assert ff.forward(ctx, h.cuda(), residual=acc) is None
    f32 = {k: v.float().numpy() for k, v in ws.items()}
    ref = res.numpy() + llama_plain.swiglu(h.float().numpy(), f32["gate_proj.weight"], f32["up_proj.weight"],
                                           f32["down_proj.weight"])
    assert np.abs(acc.cpu().numpy() - ref).max() <= tol * np.abs(ref).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout", ["half", "interleaved"])
def test_attention_part_alone(dtype, layout):
    """The mixer alone: two steps (a portion, then the rest) against the plain
    attention block over the whole sequence."""
    from garuda_b200.kernels import CudaOps
    from garuda_b200.parts import PagedAttention, LayerCache
    from garuda_b200.engine.batch import StepBatch
    ops = CudaOps("cuda:0", tensor_cores=dtype == torch.bfloat16)
    d, Hq, Hkv, hd, page, T = 72, 6, 2, 16, 8, 29
    att = PagedAttention(d, Hq, Hkv, hd, position={"name": "rotary", "params": {"theta": 10000.0, "head_dim": hd,
                                                                                 "layout": layout}}, window=11)
    ws = {k: (torch.randn(v.shape) * 0.15).to(dtype) for k, v in att.tensors().items()}
    att.load({k: v.cuda() for k, v in ws.items()}, ops, dtype)
    h = torch.randn(T, d).to(dtype)
    k_pool = torch.zeros(8, Hkv, page, hd, dtype=dtype, device="cuda")
    v_pool = torch.zeros_like(k_pool)
    bt = torch.tensor([[5, 2, 7, 0]], dtype=torch.int32).cuda()
    f32 = {"self_attn." + k: v.float().numpy() for k, v in ws.items()}
    f32["input_layernorm.weight"] = np.ones(d, dtype=np.float32)
    cfg = dict(num_attention_heads=Hq, num_key_value_heads=Hkv, head_dim=hd, rms_norm_eps=0.0,
               rope_theta=10000.0, rope_layout=layout)
    # the plain block norms its input; feed it rows of unit mean square so that the norm is the identity
    hn = h.float().numpy()
    hn = hn / np.sqrt((hn * hn).mean(-1, keepdims=True))
    att_in = torch.from_numpy(hn).to(dtype)
    outs = []
    k_pool.zero_(), v_pool.zero_()
    for start, n in ((0, 18), (18, 11)):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
        batch = StepBatch(num_tokens=n, num_requests=1, token_ids=i32([0] * n), positions=i32(list(range(start, start + n))),
                          token_req=i32([0] * n), cu_q=i32([0, n]), kv_lens=i32([start + n]), slots=i32([0]),
                          block_tables=[bt], logit_rows=i32([]), num_logit_rows=0, max_q_len=n, max_kv_len=start + n)
        cache = LayerCache(need=att.cache_need(), k=k_pool, v=v_pool, block_table=bt, page_size=page)
        outs.append(att.forward(_ctx(ops, dtype, batch), att_in[start:start + n].cuda(), cache).float().cpu())
    ref = llama_plain.attention_block(att_in.float().numpy(), f32, cfg, np.arange(T), 11)
    got = torch.cat(outs).numpy()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(got - ref).max() <= tol * np.abs(ref).max()


# ---------------------------------------------------------------------- a toy mixer
def test_a_toy_mixer_with_state_of_its_own_can_be_registered_built_and_stepped():
    """A mixer defined here, unknown to the framework: a running mean of the normed
    inputs per request, kept in a fixed-size state slot. It is registered, named
    in a layer list beside attention layers, built, and stepped in portions; the
    result must not depend on how the tokens were cut."""
    from garuda_b200.parts import (Mixer, FixedState, TensorSpec, PartSpec, BlockSpec, register_mixer)
    from garuda_b200.models.decoder import Decoder, ModelSpec, LayerCall
    from garuda_b200.cache import PagedCache, CacheConfig
    from garuda_b200.engine.step import StepRunner, StepEntry
    from garuda_b200.kernels import CudaOps
    from garuda_b200.weights.random_init import random_tensor

    @register_mixer("toy_running_mean_local")
    class RunningMean(Mixer):
        def __init__(self, width):
            self.width = width

        def tensors(self):
            return {"gain": TensorSpec((self.width,), role="vector", init=("normal_about_one", 0.1))}

        def cache_need(self):
            return FixedState((self.width + 1,), torch.float32)       # running sum, and a count

        def load(self, tensors, ops, dtype):
            super().load(tensors, ops, dtype)
            self.gain = tensors["gain"].float()

        def forward(self, ctx, h, cache, residual=None):
            b = ctx.batch
            out = torch.empty(h.shape, dtype=torch.float32, device=h.device)
            cu = b.host["cu_q"]
            for r, slot in enumerate(b.host["slots"]):
                rows = h[cu[r]:cu[r + 1]].float()
                state = cache.state[slot]
                sums = state[:-1] + torch.cumsum(rows, 0)
                counts = state[-1] + torch.arange(1, rows.shape[0] + 1, device=h.device)
                out[cu[r]:cu[r + 1]] = sums / counts[:, None] * self.gain
                state[:-1] = sums[-1]
                state[-1] = counts[-1]
            return out

    d, V = 64, 100
    attn = lambda l: PartSpec("paged_attention", dict(width=d, heads=4, kv_heads=2, head_dim=16,
                              position={"name": "rotary", "params": {"theta": 1e4, "head_dim": 16}}),
                              prefix=f"layers.{l}.attn.")
    norm = lambda p: PartSpec("rms", dict(width=d, eps=1e-5), prefix=p)
    ff = lambda l: PartSpec("swiglu", dict(width=d, inner=96), prefix=f"layers.{l}.ff.")
    layers = [BlockSpec(attn(0), ff(0), norm("layers.0.n1."), norm("layers.0.n2.")),
              BlockSpec(PartSpec("toy_running_mean_local", dict(width=d), prefix="layers.1.toy."), ff(1),
                        norm("layers.1.n1."), norm("layers.1.n2.")),
              BlockSpec(attn(2), None, norm("layers.2.n1."), None)]
    # the run order names layer 0 twice, and its second call reads the first call's cache
    spec = ModelSpec(architecture="ToyForTests", width=d, vocab_size=V, max_positions=128, embedding="embed",
                     layers=layers, order=[LayerCall(0), LayerCall(1), LayerCall(2), LayerCall(0, reads_cache_of=0)],
                     final_norm=norm("final."), head=None)
    model = Decoder(spec)
    assert len(model.state_calls) == 1 and len(model.cache_groups) == 1 and len(model.cache_groups[0].calls) == 2
    ops = CudaOps("cuda:0", tensor_cores=False)
    tensors = {n: random_tensor(0, n, ts.shape, ts.init).cuda() for n, ts in model.expected_tensors().items()}
    model.load(tensors, ops, torch.float32)
    cache = PagedCache(model, CacheConfig(page_size=8, max_tokens=256, max_requests=3, max_positions=128),
                       torch.float32, "cuda:0")
    runner = StepRunner(model, cache, ops, torch.float32, "cuda:0")
    toks = [np.random.default_rng(i).integers(0, V, 40).tolist() for i in range(2)]
    whole = [runner.run([StepEntry(i, toks[i], range(40))]).cpu().numpy().copy() for i in range(2)]
    for i in range(2):
        runner.end(i)
    # the same two requests, cut into portions and mixed in one batch, in fresh slots
    got = [[], []]
    cuts = [(0, 7, 5), (7, 2, 1), (9, 20, 30), (29, 11, 4)]
    for a_start, a_n, b_n in cuts:
        b_start = sum(c[2] for c in cuts[:cuts.index((a_start, a_n, b_n))])
        out = runner.run([StepEntry(10, toks[0][a_start:a_start + a_n], range(a_n)),
                          StepEntry(11, toks[1][b_start:b_start + b_n], range(b_n))]).cpu().numpy()
        got[0].append(out[:a_n].copy())
        got[1].append(out[a_n:].copy())
    for i in range(2):
        cut = np.concatenate(got[i])
        assert np.abs(cut - whole[i]).max() <= 2e-5 * np.abs(whole[i]).max()
    # a request that starts in a slot another one has used starts from zeroed state
    runner.end(10), runner.end(11)
    again = runner.run([StepEntry(12, toks[0], range(40))]).cpu().numpy()
    assert np.abs(again - whole[0]).max() <= 2e-5 * np.abs(whole[0]).max()
