"""Fasesun on the GPU against the plain statement in `plain_fasesun.py`: each mechanism alone (kernels and one-layer models),
whole prompts, single tokens, portions, unequal batches, slots and pages that are used again, page borders, long decoding,
odd sizes, greedy generation through `generate()` and the trace replay as a subprocess."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import fasesun_models as fm
import plain_fasesun as plain
from helpers import relative_error, run_batched, run_tail_stepwise, run_whole
from tau_rs_b200 import Engine, StepEntry, generate, load_model

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOLERANCE = {"float32": 2e-5, "bfloat16": 2e-2}
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def close(found, wanted, dtype) -> bool:
    """float32: every logit within 2e-5 of the largest.  bfloat16: half of the positions within 1.5e-2 and nine in ten within
    5e-2 (two roundings of the looped model itself differ by 0.6e-2 at the median and 1.2e-2 at nine in ten); roundings move a
    router's scores, and where two experts were a close call the library and the plain statement may choose differently at a
    position, which says nothing about either (the float32 runs pin every choice)."""
    if dtype == "float32":
        return relative_error(found, wanted) < TOLERANCE[dtype]
    rows = (found.double() - wanted.double()).abs().amax(dim=-1) / wanted.double().abs().max()
    return float(rows.median()) < 1.5e-2 and float(torch.quantile(rows, 0.9)) < 5e-2


def tokens_for(cfg, count, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=count).tolist()


def plain_logits(cfg, values, tokens, dtype):
    rounding = plain.bfloat16_rounding if dtype == "bfloat16" else plain.no_rounding
    return plain.forward(cfg, values, tokens, rounding).float()


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("fasesun")
    made = {}
    for name, cfg, seed in (("mixed", fm.MIXED, 11), ("odd", fm.ODD, 12), ("peaky", fm.PEAKY, 13), ("ragged", fm.RAGGED, 14)):
        folder = str(root / name)
        made[name] = (folder, cfg, fm.write_model(folder, cfg, seed))
    return made


def engine_of(models, name, dtype, max_tokens=1024):
    folder, cfg, values = models[name]
    return Engine(load_model(folder, dtype, "gpu"), max_tokens), cfg, values


# ---- each mechanism alone ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", [
    fm.latent(mlp=None), fm.latent(heads=1, dim=8, rot_dim=24, rot_dims=12, vdim=8, q_rank=16, kv_rank=16, scale=0.9, mlp=None),
    fm.latent(heads=3, dim=32, rot_dim=16, rot_dims=16, vdim=40, q_rank=24, kv_rank=56, mlp=None),
    fm.latent(heads=2, dim=16, rot_dim=16, vdim=16, q_rank=16, kv_rank=800, mlp=None),
    fm.mlstm(mlp=None), fm.mlstm(heads=3, dim=8, vdim=130, gate_cap=2.0, mlp=None),
    fm.lightning(mlp=None), fm.lightning(heads=2, dim=100, vdim=12, decay=[0.3, 1.0], mlp=None),
], ids=["latent", "latent_one_head", "latent_expanding", "latent_wide_rank", "mlstm", "mlstm_wide_values", "lightning", "lightning_wide_keys"])
def test_a_mixer_alone(tmp_path, layer, dtype):
    cfg = fm.config([layer], width=80, vocab=61)
    values = fm.write_model(str(tmp_path), cfg, 5)
    engine = Engine(load_model(str(tmp_path), dtype, "gpu"), 512)
    tokens = tokens_for(cfg, 150, 3)
    wanted = plain_logits(cfg, values, tokens, dtype)
    assert relative_error(run_whole(engine, tokens), wanted) < TOLERANCE[dtype]
    assert relative_error(run_tail_stepwise(engine, tokens, 149), wanted[1:]) < TOLERANCE[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts, top, softmax, renormalize, shared", [(6, 3, False, False, True), (1, 1, False, False, True), (5, 5, False, True, False),
                                                                        (40, 2, True, True, True), (7, 1, True, False, False)])
def test_routed_experts_kernels(dtype, experts, top, softmax, renormalize, shared):
    from tau_rs_b200.csrc import kernels

    torch.manual_seed(experts * 10 + top)
    tokens, width, inner, device, kind = 37, 72, 40, "cuda", TORCH[dtype]
    rounding = plain.bfloat16_rounding if dtype == "bfloat16" else plain.no_rounding
    hidden = rounding(torch.randn(tokens, width))
    W = {"m.router": torch.randn(experts, width) * 0.3, "m.correction": torch.randn(experts) * 0.5, "m.shared.sg": torch.randn(1, width) * 0.2}
    for expert in range(experts):
        W[f"m.e{expert}.gate"], W[f"m.e{expert}.up"] = rounding(torch.randn(inner, width) / 8), rounding(torch.randn(inner, width) / 8)
        W[f"m.e{expert}.down"] = rounding(torch.randn(width, inner) / 6)
    # The plain router: scores, choice with the correction, weights without it.
    z = hidden.double() @ W["m.router"].double().T
    scores = torch.softmax(z, dim=-1) if softmax else torch.sigmoid(z)
    picked = torch.topk(scores + W["m.correction"].double(), top, dim=-1).indices
    weight = torch.gather(scores, 1, picked)
    if renormalize:
        weight = weight / weight.sum(dim=-1, keepdim=True)
    shared_out = rounding(torch.randn(tokens, width)) if shared else None
    shared_gate = torch.sigmoid(hidden.double() @ W["m.shared.sg"].double().T)[:, 0]
    wanted = torch.zeros(tokens, width, dtype=torch.float64)
    for token in range(tokens):
        for place in range(top):
            wanted[token] += weight[token, place] * plain.gated_expert(hidden[token : token + 1].double(), W, f"m.e{int(picked[token, place])}", rounding)[0]
        if shared:
            wanted[token] += shared_gate[token] * shared_out[token].double()
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=device)
    gate = torch.empty(tokens, dtype=torch.float32, device=device)
    x = hidden.to(device, kind)
    kernels.moe_route(x, W["m.router"].to(device), W["m.correction"].to(device), W["m.shared.sg"].reshape(-1).to(device) if shared else None, chosen, weights,
                      gate if shared else None, top, softmax, renormalize)
    assert torch.equal(chosen.cpu().long().sort(dim=-1).values, picked.sort(dim=-1).values)
    order = chosen.cpu().long()
    assert torch.allclose(weights.cpu().double(), (torch.gather(scores, 1, order) / (torch.gather(scores, 1, order).sum(-1, keepdim=True) if renormalize else 1.0)), atol=1e-5)
    gate_up = torch.stack([torch.cat([W[f"m.e{e}.gate"], W[f"m.e{e}.up"]]) for e in range(experts)]).to(device, kind)
    down = torch.stack([W[f"m.e{e}.down"] for e in range(experts)]).to(device, kind)
    inner_values = torch.empty((tokens, top, inner), dtype=kind, device=device)
    kernels.moe_gate_up(x, gate_up, chosen, inner_values)
    out = torch.empty((tokens, width), dtype=torch.float32, device=device)
    kernels.moe_down(inner_values, down, chosen, weights, shared_out.to(device, kind) if shared else None, gate if shared else None, out)
    assert relative_error(out.cpu(), wanted) < (1e-5 if dtype == "float32" else 1e-2)


def test_grouped_experts_equal_streamed_experts():
    """A run of new tokens in bfloat16 takes the grouped products; the same tokens through the streaming kernels differ by
    roundings of the products alone, and every token's chosen experts are the same."""
    from types import SimpleNamespace

    from tau_rs_b200.config import RoutedExpertsSpec, SwiGLUSpec
    from tau_rs_b200.parts import routed_experts

    torch.manual_seed(3)
    width, inner, experts, top, tokens = 64, 24, 7, 3, 400
    names = dict(gate_name="gate", up_name="up", down_name="down", weight_suffix="")
    spec = RoutedExpertsSpec(hidden=width, intermediate=inner, experts=experts, top=top, shared=SwiGLUSpec(hidden=width, intermediate=16, **names), shared_gate=True)
    part = routed_experts.RoutedExperts(spec, "m", torch.bfloat16, "cuda")
    assert part.interleave
    W = {}
    for name, tensor_spec in part.tensor_specs().items():
        value = torch.randn(*tensor_spec.shape) / (tensor_spec.shape[-1] ** 0.5 if len(tensor_spec.shape) > 1 else 1.0)
        W[name] = value.bfloat16().float()
        part.assign(name, value.to("cuda", torch.bfloat16 if tensor_spec.role == "matrix" else torch.float32))
    part.finalize_weights()
    hidden = torch.randn(tokens, width).bfloat16()
    grouped = part.forward(hidden.cuda(), SimpleNamespace(all_single=False)).cpu()
    streamed = part.forward(hidden.cuda(), SimpleNamespace(all_single=True)).cpu()
    assert relative_error(grouped, streamed) < 1e-2
    wanted = plain.mixture_of_experts(hidden.double(), W, "m", {"router": {"experts": experts, "top": top}, "shared": {"ff": 16}}, plain.bfloat16_rounding)
    rows = (grouped.double() - wanted).abs().amax(dim=-1) / wanted.abs().max()
    assert float(torch.quantile(rows, 0.95)) < 1e-2           # a close call of the router may flip at a few tokens


def test_the_32_bit_stream_kernels():
    from tau_rs_b200.csrc import kernels

    torch.manual_seed(0)
    rows, width, device = 19, 100, "cuda"
    stream = torch.randn(rows, width) * 30
    a, b = torch.randn(rows, width).bfloat16(), torch.randn(rows, width)
    weight = 1 + 0.2 * torch.randn(width)
    total = stream.double() + (a.double() + b.double())
    wanted = plain.rms_norm(total, weight.double(), 1e-5)
    on_device = stream.to(device)
    out = torch.empty((rows, width), dtype=torch.bfloat16, device=device)
    kernels.stream_add_norm(on_device, (a.to(device), b.to(device)), weight.to(device), 1e-5, out)
    assert torch.allclose(on_device.cpu().double(), total, atol=1e-5)            # the sum stays 32-bit: no bfloat16 step of 0.25 at 30
    assert relative_error(out.cpu(), wanted) < 5e-3
    picked = torch.tensor([4, 0, 18], dtype=torch.int32, device=device)
    gathered = torch.empty((3, width), dtype=torch.float32, device=device)
    kernels.stream_add_norm(on_device, None, weight.to(device), 1e-5, gathered, rows=picked, update=False)
    assert relative_error(gathered.cpu(), wanted[[4, 0, 18]]) < 1e-5
    table = torch.randn(50, width).bfloat16()
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device=device)
    embedded = torch.empty((4, width), dtype=torch.float32, device=device)
    kernels.embedding(ids, table.to(device), embedded)
    assert torch.equal(embedded.cpu(), table[[3, 49, 0, 3]].float())
    values, gate = torch.randn(rows, 6 * 14) * 5, torch.randn(rows, 200)
    for groups, normalize in ((6, True), (1, True), (1, False)):
        base = plain.rms_norm(values.double().view(rows, groups, -1), None, 1e-5).reshape(rows, -1) if normalize else values.double()
        wanted = base * weight[:84].double() * torch.sigmoid(gate[:, 100:184].double())
        out = torch.empty((rows, 84), dtype=torch.float32, device=device)
        kernels.gated_group_norm(values.to(device), weight[:84].contiguous().to(device), gate.to(device)[:, 100:184], out, groups, 1e-5, normalize)
        assert relative_error(out.cpu(), wanted) < 1e-5


def test_products_of_a_batch_of_heads():
    from tau_rs_b200.csrc import kernels

    torch.manual_seed(1)
    rows, heads, depth, features = 70, 5, 24, 72
    whole = torch.randn(rows, heads, depth + 8).cuda()
    weight = torch.randn(heads, features, depth).cuda()
    out = torch.zeros(rows, heads, features + 3).cuda()
    kernels.gemm_simt_batched(whole[:, :, :depth], weight, out[:, :, :features])
    wanted = torch.einsum("rhk,hnk->rhn", whole[:, :, :depth].double().cpu(), weight.double().cpu())
    assert relative_error(out[:, :, :features].cpu(), wanted) < 1e-5 and float(out[:, :, features:].abs().sum()) == 0.0


# ---- whole models: cuttings, batches, reuse --------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "ragged"])
def test_whole_prompts_single_tokens_and_the_first_positions(models, name, dtype):
    engine, cfg, values = engine_of(models, name, dtype)
    tokens = tokens_for(cfg, 200, 21)
    wanted = plain_logits(cfg, values, tokens, dtype)
    whole = run_whole(engine, tokens)
    assert close(whole, wanted, dtype)
    assert close(whole[:3], wanted[:3], dtype)               # the first tokens: empty state, the sink almost alone
    assert close(run_whole(engine, tokens[:1]), wanted[:1], dtype)
    stepwise = run_tail_stepwise(engine, tokens, 199)                              # every token but the first alone, through the graphs
    assert close(stepwise, wanted[1:], dtype)
    if dtype == "float32":
        assert relative_error(stepwise, whole[1:]) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens_and_page_borders(models, dtype):
    engine, cfg, values = engine_of(models, "mixed", dtype)
    tokens = tokens_for(cfg, 330, 22)
    wanted = plain_logits(cfg, values, tokens, dtype)
    slot = engine.open_sequence()
    found, position = [], 0
    for count in [2, 2, 3, 56, 1, 1, 62, 2, 64, 1, 63, 2, 5, 64, 2]:               # runs that end at, before and behind positions 63/64, 127/128, ...
        piece = tokens[position : position + count]
        found.append(engine.step([StepEntry(slot, piece, list(range(count)))]).float().cpu().clone())
        position += count
    assert position == 330
    engine.close_sequence(slot)
    assert close(torch.cat(found), wanted, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_sharp_softmax_loses_no_key_far_away_or_at_a_page_border(models, dtype):
    engine, cfg, values = engine_of(models, "peaky", dtype)
    tokens = tokens_for(cfg, 400, 23)
    wanted = plain_logits(cfg, values, tokens, dtype)
    assert close(run_whole(engine, tokens), wanted, dtype)
    tail = run_tail_stepwise(engine, tokens, 150)                                  # decoded queries cross the borders at 256 and 320
    assert close(tail, wanted[-150:], dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "peaky", "ragged"])
def test_unequal_batches_against_each_request_alone(models, name, dtype):
    engine, cfg, values = engine_of(models, name, dtype, 2048)
    lengths, prompts = [90, 31, 140, 5, 66], [70, 1, 129, 3, 64]
    requests = [tokens_for(cfg, length, 30 + index) for index, length in enumerate(lengths)]
    together = run_batched(engine, requests, prompts)
    for request, prompt, rows in zip(requests, prompts, together):
        wanted = plain_logits(cfg, values, request, dtype)[prompt - 1 :]
        assert close(rows, wanted, dtype)
    engine.cache.check()
    assert engine.cache.slots.in_use == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_sequences_of_wide_heads(tmp_path, dtype):
    """Enough (sequence, head, column tile) blocks that the state kernel takes its wider tiles; each request equals itself alone."""
    cfg = fm.config([fm.mlstm(heads=3, dim=8, vdim=130, gate_cap=3.0, mlp=None), fm.lightning(heads=4, dim=24, vdim=70, mlp=None)], width=64, vocab=83)
    values = fm.write_model(str(tmp_path), cfg, 9)
    engine = Engine(load_model(str(tmp_path), dtype, "gpu"), 64 * 16)
    requests = [tokens_for(cfg, 20 + 3 * index, 90 + index) for index in range(14)]
    together = run_batched(engine, requests, [len(request) - 4 for request in requests])
    for request, rows in zip(requests, together):
        assert close(rows, plain_logits(cfg, values, request, dtype)[len(request) - 5 :], dtype)


def test_slots_and_pages_that_are_used_again_start_clean(models):
    """A cache of three pages and as many slots: every request takes a slot whose state another left behind and pages that
    another wrote."""
    engine, cfg, values = engine_of(models, "mixed", "float32", 64 * 3)
    for round_number in range(4):
        requests = [tokens_for(cfg, length, 40 + 3 * round_number + index) for index, length in enumerate([60 + round_number, 40, 17])]
        together = run_batched(engine, requests, [len(request) - 6 for request in requests])
        for request, rows in zip(requests, together):
            assert relative_error(rows, plain_logits(cfg, values, request, "float32")[len(request) - 7 :]) < TOLERANCE["float32"]
        engine.cache.check()
    long_one = tokens_for(cfg, 190, 50)
    assert relative_error(run_whole(engine, long_one), plain_logits(cfg, values, long_one, "float32")) < TOLERANCE["float32"]


def test_long_decoding_in_bfloat16_stays_with_the_plain_statement(models):
    engine, cfg, values = engine_of(models, "mixed", "bfloat16")
    tokens = tokens_for(cfg, 420, 24)
    wanted = plain_logits(cfg, values, tokens, "bfloat16")
    assert close(run_tail_stepwise(engine, tokens, 400), wanted[-400:], "bfloat16")


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_greedy_generation_through_the_library_entry_point(models, name):
    folder, cfg, values = models[name]
    prompts = [tokens_for(cfg, length, 60 + index) for index, length in enumerate([9, 30, 2])]
    output = generate(folder, prompts, max_new_tokens=12, dtype="float32", stop_tokens=[])
    for prompt, result in zip(prompts, output):
        tokens = list(prompt)
        for _ in range(12):
            logits = plain_logits(cfg, values, tokens, "float32")[-1]
            best, second = torch.topk(logits, 2).values
            if float(best - second) < 1e-3 * float(logits.abs().max()):
                break                                                                # a close call proves nothing either way
            tokens.append(int(torch.argmax(logits)))
        made = len(tokens) - len(prompt)
        assert list(result.tokens[:made]) == tokens[len(prompt) :] and made >= 1


def test_trace_replay_of_a_fasesun_folder(models, tmp_path):
    folder, cfg, values = models["odd"]
    first, second = tokens_for(cfg, 70, 70), tokens_for(cfg, 33, 71)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": first[:66], "want": [0, 65]}, {"id": "b", "tokens": second[:30], "want": [29]}], "end": []}]
    for index in range(3):
        steps.append({"step": index + 1, "entries": [{"id": "a", "tokens": [first[66 + index]], "want": [0]}, {"id": "b", "tokens": [second[30 + index]], "want": [0]}],
                      "end": ["b"] if index == 2 else []})
    steps.append({"step": 4, "entries": [{"id": "a", "tokens": [first[69]], "want": []}], "end": ["a"]})
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out), "--max-tokens", "256"],
                          input="\n".join(json.dumps(step) for step in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.split("\n") if line.startswith("done")] == [f"done {index}" for index in range(5)]
    wanted_a, wanted_b = plain_logits(cfg, values, first, "float32"), plain_logits(cfg, values, second, "float32")
    rows = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, cfg["vocab"])
    assert relative_error(torch.from_numpy(rows), torch.stack([wanted_a[0], wanted_a[65], wanted_b[29]])) < TOLERANCE["float32"]
    rows = np.fromfile(out / "3.f32", dtype="<f4").reshape(2, cfg["vocab"])
    assert relative_error(torch.from_numpy(rows), torch.stack([wanted_a[68], wanted_b[32]])) < TOLERANCE["float32"]
    assert not (out / "4.f32").exists()


def test_the_command_line_on_a_fasesun_folder(models, tmp_path):
    """`bin/tau` on a Fasesun folder: greedy tokens in 32-bit equal those of `generate()`, with graphs and without, in chunks of
    prompt tokens; bfloat16 runs from the same folder (the design stores bfloat16, so a folder need not say so); random
    weights are written for a Fasesun config.json and read back."""
    folder, cfg, values = models["mixed"]
    prompts = [tokens_for(cfg, 40, 80), tokens_for(cfg, 7, 81)]
    wanted = [list(result.tokens) for result in generate(folder, prompts, max_new_tokens=8, dtype="float32", stop_tokens=[])]

    def run(arguments):
        done = subprocess.run([os.path.join(ROOT, "bin", "tau")] + arguments, capture_output=True, text=True, timeout=900)
        assert done.returncode == 0, done.stderr[-2000:]
        return [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]

    base = ["--model", folder, "--max-tokens", "8", "--stop-ids", ""]
    for prompt in prompts:
        base += ["--prompt-ids", ",".join(str(token) for token in prompt)]
    records = run(base + ["--dtype", "f32"])
    assert [record["tokens"] for record in records if "tokens" in record] == wanted
    records = run(base + ["--dtype", "f32", "--cuda-graph", "none", "--prefill-chunk-size", "16"])
    assert [record["tokens"] for record in records if "tokens" in record] == wanted
    records = run(base + ["--dtype", "bf16"])
    assert all(len(record["tokens"]) == 8 for record in records if "tokens" in record)
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(fm.PEAKY))
    drawn = str(tmp_path / "drawn")
    records = run(["--random-weights", str(config_path), "--model", drawn, "--seed", "4", "--max-tokens", "5", "--stop-ids", "", "--prompt-ids", "1,2,3"])
    assert [len(record["tokens"]) for record in records if "tokens" in record] == [5]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_window_on_latent_attention_in_another_design(tmp_path, dtype):
    """The mixer's spec takes a window that Fasesun never sets.  A toy architecture sets it: position i then sees the last 70
    positions only, in whole prompts (the expanded form in bfloat16), in portions and in single tokens, and the cache gives the
    pages back that fell out of it."""
    import dataclasses

    from tau_rs_b200.config import FasesunConfig, register_architecture
    from tau_rs_b200.config.registry import unregister_architecture
    from tau_rs_b200.models.fasesun import build_fasesun_spec

    window = 70

    def parse(raw):
        return FasesunConfig.from_json(dict(raw, architecture="Fasesun"))

    def build(config):
        spec = build_fasesun_spec(config)
        blocks = tuple(dataclasses.replace(block, mixer=dataclasses.replace(block.mixer, window=window)) for block in spec.blocks)
        return dataclasses.replace(spec, architecture="WindowedLatentToy", blocks=blocks)

    register_architecture("WindowedLatentToy", "windowedlatenttoy", parse, build, storage_dtype="bfloat16")
    try:
        layers = [fm.latent(heads=3, dim=16, rot_dim=16, vdim=24, q_rank=32, kv_rank=48, scale=1.5, mlp=None),
                  fm.latent(heads=2, dim=24, rot_dim=16, vdim=8, q_rank=16, kv_rank=36, scale=1.0, mlp=None)]
        cfg = dict(fm.config(layers, width=64, vocab=97), architecture="WindowedLatentToy")
        values = fm.write_model(str(tmp_path), cfg, 17)
        plain_cfg = {**cfg, "layers": [{**layer, "mixer": {**layer["mixer"], "window": window}} for layer in layers]}
        tokens = tokens_for(cfg, 300, 18)
        wanted = plain_logits(plain_cfg, values, tokens, dtype)
        engine = Engine(load_model(str(tmp_path), dtype, "gpu"), 64 * 6)
        assert close(run_whole(engine, tokens), wanted, dtype)
        slot = engine.open_sequence()
        found, position = [], 0
        for count in [150, 3, 64, 2] + [1] * 81:
            piece = tokens[position : position + count]
            found.append(engine.step([StepEntry(slot, piece, list(range(count)))]).float().cpu().clone())
            position += count
            engine.cache.check()
        assert position == 300 and all(len(group.held[slot]) <= 3 for group in engine.cache.kv.values())
        engine.close_sequence(slot)
        assert close(torch.cat(found), wanted, dtype)
    finally:
        unregister_architecture("WindowedLatentToy")
