"""Bisudra on the GPU against the plain statement in `plain_bisudra.py`: each mechanism's kernels alone, then whole models: whole
prompts, single tokens, portions, unequal batches, slots and pages that are used again, windows' edges and page borders, keys
far back, long decoding, odd sizes, greedy generation through `generate()`, the command line and the trace replay."""
import json
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import bisudra_models as bm
import plain_bisudra as plain
from helpers import relative_error, run_batched, run_tail_stepwise, run_whole
from tau_rs_b200 import Engine, StepEntry, generate, load_model

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOLERANCE = {"float32": 5e-5, "bfloat16": 4e-2}
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEVICE = "cuda"


def close(found, wanted, dtype) -> bool:
    """float32: every logit within 5e-5 of the largest.  bfloat16 (the plain statement rounds nothing): half of the positions within
    2e-2 of the largest logit and nine in ten within 6e-2; where two experts were a close call the library and the plain statement
    may choose differently at a position, which says nothing about either (the float32 runs pin every choice)."""
    if dtype == "float32":
        return relative_error(found, wanted) < TOLERANCE[dtype]
    rows = (found.double() - wanted.double()).abs().amax(dim=-1) / wanted.double().abs().max()
    return float(rows.median()) < 2e-2 and float(torch.quantile(rows, 0.9)) < 6e-2


def tokens_for(cfg, count, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=count).tolist()


_PLAIN = {}


def plain_logits(cfg, values, tokens):
    key = (id(values), tuple(tokens))
    if key not in _PLAIN:
        _PLAIN[key] = plain.forward(tokens, {name: value.double() for name, value in values.items()}, cfg).float()
    return _PLAIN[key]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("bisudra")
    made = {}
    for name, cfg, seed in (("mixed", bm.MIXED, 11), ("odd", bm.ODD, 12), ("one_tap", bm.ONE_TAP, 13), ("peaky", bm.PEAKY, 14), ("edgy", bm.EDGY, 15)):
        folder = str(root / name)
        made[name] = (folder, cfg, bm.write_model(folder, cfg, seed))
    return made


def engine_of(models, name, dtype, max_tokens=1024):
    folder, cfg, values = models[name]
    return Engine(load_model(folder, dtype, "gpu"), max_tokens), cfg, values


def on_device(tensor, dtype=torch.float32):
    return tensor.to(DEVICE, dtype).contiguous()


def packed_step(runs, slots):
    """The metadata of a step in which sequence i brings `runs[i]` tokens and sits in cache slot `slots[i]`."""
    bounds = np.concatenate([[0], np.cumsum(runs)]).astype(np.int32)
    token_seq = np.concatenate([np.full(count, index, dtype=np.int32) for index, count in enumerate(runs)])
    as_device = lambda values: torch.tensor(np.asarray(values, dtype=np.int32), device=DEVICE)
    return SimpleNamespace(n_seqs=len(runs), token_seq=as_device(token_seq), cu_seqlens=as_device(bounds), seq_slot=as_device(slots),
                           all_single=all(count == 1 for count in runs))


# ---- each mechanism's kernels alone -----------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_causal_taps_carry_their_tail_from_step_to_step(dtype, taps):
    """Three sequences in slots 5, 0 and 2 of a state that held other values; runs of 1, 2 and many tokens, shorter and longer than
    the tail, over four steps: every step equals the plain convolution of the whole sequence so far."""
    from tau_rs_b200.csrc import kernels

    torch.manual_seed(taps)
    width, slots = 52, [5, 0, 2]
    weight = torch.randn(width, taps, dtype=torch.float64)
    state = torch.randn(7, max(taps - 1, 1), width, device=DEVICE)[:, : taps - 1].contiguous() if taps > 1 else None
    if state is not None:
        state[slots] = 0.0          # a sequence starts from zeros, as the cache leaves a slot
    history = [torch.zeros(0, width, dtype=torch.float64) for _ in slots]
    for runs in ([1, 9, 2], [1, 1, 1], [1, 1, 1], [2, 1, 6], [1, 1, 1], [5, 2, 1]):      # steps of single tokens move the state in the same launch
        new = [torch.randn(count, width, dtype=torch.float64).float().double() for count in runs]
        x = on_device(torch.cat(new))
        read = torch.empty(x.shape, dtype=TORCH[dtype], device=DEVICE)
        rounded = torch.empty_like(read)
        kernels.causal_taps(x, on_device(weight.T), state, packed_step(runs, slots), read, rounded)      # the kernel wants [taps, width]
        wanted = []
        for index, rows in enumerate(new):
            history[index] = torch.cat([history[index], rows])
            wanted.append((history[index] + plain.causal_taps(history[index], weight))[-rows.shape[0] :])
        assert relative_error(read.float().cpu(), torch.cat(wanted)) < (1e-6 if dtype == "float32" else 5e-3)
        assert torch.equal(rounded.float().cpu(), x.cpu().to(TORCH[dtype]).float())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("centred, biased, gated", [(True, True, True), (True, True, False), (False, False, True)])
def test_the_gated_sum_behind_a_norm(dtype, centred, biased, gated):
    from tau_rs_b200.csrc import kernels

    torch.manual_seed(3)
    rows, width, eps = 19, 203, 1e-3
    stream, branch = torch.randn(rows, width), (3.0 + 2.0 * torch.randn(rows, width)).to(TORCH[dtype]).float()
    gate = torch.randn(rows, width + 5).to(TORCH[dtype]).float()
    weight, bias = torch.randn(width), torch.randn(width)
    y = branch.double() * (torch.sigmoid(gate[:, :width].double()) if gated else 1.0)
    normed = plain.layer_norm(y, weight.double(), bias.double() if biased else 0.0, eps) if centred else plain.unit_rms(y, eps) * weight.double()
    if not centred and biased:
        normed = normed + bias.double()
    wanted = stream.double() + normed
    source, target = on_device(stream), torch.empty(rows, width, device=DEVICE)
    copy = torch.empty(rows, width, dtype=TORCH[dtype], device=DEVICE)
    arguments = (on_device(branch, TORCH[dtype]), on_device(gate, TORCH[dtype])[:, :width] if gated else None, on_device(weight), on_device(bias) if biased else None, eps, centred)
    kernels.gated_add_norm(source, target, *arguments, copy)
    assert relative_error(target.cpu(), wanted) < 2e-6 and torch.equal(source.cpu(), stream)
    assert torch.equal(copy.float().cpu(), target.cpu().to(TORCH[dtype]).float())
    kernels.gated_add_norm(source, source, *arguments)                      # in place, from a 32-bit branch as well
    assert torch.equal(source, target)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_side_input_and_the_mix_of_results(dtype):
    from tau_rs_b200.csrc import kernels

    torch.manual_seed(4)
    rows, width, dim, vocab, eps = 23, 77, 6, 31, 1e-4
    kind = TORCH[dtype]
    z, table = torch.randn(rows, dim).to(kind).float() * 2, torch.randn(vocab, 4 * dim).to(kind).float()
    token_ids = torch.randint(0, vocab, (rows,), dtype=torch.int32)
    out = torch.empty(rows, dim, dtype=kind, device=DEVICE)
    kernels.side_gate(on_device(z, kind), on_device(table, kind), token_ids.to(DEVICE), 2 * dim, out)
    wanted = plain.gelu_tanh(z.double()) * table.double()[token_ids.long(), 2 * dim : 3 * dim]
    assert relative_error(out.float().cpu(), wanted) < (1e-6 if dtype == "float32" else 5e-3)
    # x + y / rms(y) * w as the newest of four results, then their mix; and without a mix, in place.
    results = torch.randn(5, rows, width)
    y, weight, mix = torch.randn(rows, width) * 3, torch.randn(width), torch.randn(4)
    newest = results[3].double() + plain.unit_rms(y.double(), eps) * weight.double()
    mixed = sum(mix[j].double() * results[j].double() for j in range(3)) + mix[3].double() * newest
    held, out = on_device(results), torch.empty(rows, width, device=DEVICE)
    kernels.unit_add_mix(held[3], on_device(y), on_device(weight), eps, held[3], held, on_device(mix), out)
    assert relative_error(held[3].cpu(), newest) < 2e-6 and relative_error(out.cpu(), mixed) < 2e-6
    assert torch.equal(held[4].cpu(), results[4]) and torch.equal(held[:3].cpu(), results[:3])
    alone = on_device(results[0])
    kernels.unit_add_mix(alone, on_device(y), on_device(weight), eps, alone)
    assert relative_error(alone.cpu(), results[0].double() + plain.unit_rms(y.double(), eps) * weight.double()) < 2e-6
    first = torch.empty(rows, width, device=DEVICE)
    kernels.unit_add_mix(held[0], None, None, 0.0, held[0], held, on_device(mix[:1]), first)      # one result: the embedding output alone
    assert relative_error(first.cpu(), mix[0].double() * results[0].double()) < 2e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_norm_of_chosen_rows_and_the_squared_relu(dtype):
    from tau_rs_b200.csrc import kernels

    torch.manual_seed(5)
    values, weight, bias = 4.0 + torch.randn(30, 150), torch.randn(150), torch.randn(150)
    rows = torch.tensor([29, 0, 7, 7], dtype=torch.int32)
    out = torch.empty(4, 150, dtype=TORCH[dtype], device=DEVICE)
    kernels.norm_rows(on_device(values), rows.to(DEVICE), on_device(weight), on_device(bias), 1e-5, True, out)
    wanted = plain.layer_norm(values.double()[rows.long()], weight.double(), bias.double(), 1e-5)
    assert relative_error(out.float().cpu(), wanted) < (2e-6 if dtype == "float32" else 5e-3)
    z = torch.randn(11, 37).to(TORCH[dtype])
    squared = torch.empty_like(z, device=DEVICE)
    kernels.relu_squared(z.to(DEVICE), squared)
    assert relative_error(squared.float().cpu(), torch.relu(z.double()) ** 2) < (1e-6 if dtype == "float32" else 5e-3)


@pytest.mark.parametrize("experts, top", [(6, 2), (1, 1), (5, 5), (40, 3)])
def test_a_router_with_a_bias_weighs_by_the_softmax_of_the_chosen_logits(experts, top):
    from tau_rs_b200.csrc import kernels

    torch.manual_seed(experts)
    tokens, width = 29, 72
    hidden, router, bias = torch.randn(tokens, width), torch.randn(experts, width) * 0.3, torch.randn(experts) * 2.0
    logits = hidden.double() @ router.double().T + bias.double()
    picked = torch.topk(logits, top, dim=-1).indices
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=DEVICE)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=DEVICE)
    kernels.moe_route(on_device(hidden), on_device(router), None, None, chosen, weights, None, top, True, True, on_device(bias))
    assert torch.equal(chosen.cpu().long(), picked)                        # largest first, as the plain statement lists them
    assert torch.allclose(weights.cpu().double(), torch.softmax(torch.gather(logits, 1, picked), dim=-1), atol=1e-6)
    without = torch.empty_like(chosen)
    kernels.moe_route(on_device(hidden), on_device(router), None, None, without, weights, None, top, True, True)
    assert experts == top or not torch.equal(without, chosen)                # the bias moves the choice


def attention_cache(mixer, pages, dtype, fill):
    """Pages for one layer in the layout that the sizes choose: keys and values of ordinary heads where max(dim, vdim) is a multiple
    of 16 up to 256, else one row per position."""
    kv_heads, dim, vdim = mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    wide = max(dim, vdim)
    if wide % 16 == 0 and wide <= 256:
        return tuple(torch.full((pages, 2 * kv_heads, 64, wide), fill, dtype=TORCH[dtype], device=DEVICE) for _ in range(2))
    return torch.full((pages, 64, kv_heads * (2 * dim + vdim)), fill, dtype=TORCH[dtype], device=DEVICE)


def run_attention_kernels(h, W, mixer, eps, dtype, positions, page_of, cache):
    """`h` [tokens, width] of one sequence through the stacked projection in 64-bit, then the library's kernels over a paged cache
    whose pages are `page_of[position // 64]`, in the layout of `cache` (see `attention_cache`)."""
    from tau_rs_b200.csrc import kernels

    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    stacked = torch.cat([W["m.q"], W["m.k"], W["m.v"], W["m.g"]]).double()
    projected = on_device(h.double() @ stacked.T, TORCH[dtype])
    tokens = h.shape[0]
    rotary = mixer["rot"]["dims"]
    inv_freq = torch.tensor([mixer["rot"]["base"] ** (-2.0 * i / rotary) for i in range(rotary // 2)], dtype=torch.float64).float().to(DEVICE) if rotary else None
    as_device = lambda values: torch.tensor(values, dtype=torch.int32, device=DEVICE)
    step = SimpleNamespace(positions=as_device(positions), token_seq=torch.zeros(tokens, dtype=torch.int32, device=DEVICE), n_seqs=1, all_single=tokens == 1,
                           decode_splits=0, max_len=positions[-1] + 1, cu_seqlens=as_device([0, tokens]), seq_start=as_device([positions[0]]),
                           seq_len=as_device([positions[-1] + 1]))
    pages = as_device([page_of])
    out = torch.empty((tokens, heads * vdim), dtype=TORCH[dtype], device=DEVICE)
    lam = float(torch.exp((W["m.lq1"].double() * W["m.lk1"].double()).sum()) - torch.exp((W["m.lq2"].double() * W["m.lk2"].double()).sum())) + mixer["diff"]
    gate = projected[:, heads * 2 * dim + kv_heads * (2 * dim + vdim) :]
    norms = (on_device(W["m.q.norm"]), on_device(W["m.k.norm"]), eps, inv_freq, rotary)
    if isinstance(cache, tuple):
        wide = max(dim, vdim)
        queries = torch.empty((tokens, 2 * heads, wide), dtype=TORCH[dtype], device=DEVICE)
        kernels.diff_prepare_wide(projected, *norms, queries, cache[0], cache[1], step.positions, step.token_seq, pages, heads, kv_heads, dim, vdim)
        attended = torch.empty((tokens, 2 * heads * wide), dtype=TORCH[dtype], device=DEVICE)
        kernels.attention(queries.view(tokens, -1), cache[0], cache[1], attended, step, pages, 2 * heads, 2 * kv_heads, wide, mixer["scale"], mixer["mask"]["size"])
        kernels.diff_combine(attended.view(tokens, 2 * heads, wide), gate, out, heads, kv_heads, vdim, lam, eps, 1.0 - mixer["diff"])
    else:
        queries = torch.empty((tokens, heads, 2, dim), dtype=TORCH[dtype], device=DEVICE)
        kernels.diff_prepare(projected, *norms, queries, cache, step.positions, step.token_seq, pages, heads, kv_heads, dim, vdim)
        kernels.diff_attention(queries, cache, gate, out, step, pages, kv_heads, vdim, mixer["scale"], mixer["mask"]["size"], lam, eps, 1.0 - mixer["diff"])
    return out.float().cpu()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, rot_dims", [(4, 2, 16, 24, 37, 8), (1, 1, 12, 150, 1, 6), (9, 3, 10, 6, 64, 10), (2, 1, 24, 40, 1000, 0),
                                                                          (4, 2, 16, 32, 37, 8), (2, 1, 64, 128, 100, 32), (3, 3, 48, 16, 64, 48), (8, 1, 32, 64, 1, 2), (2, 1, 32, 160, 50, 32), (1, 1, 16, 320, 40, 4)])
def test_differential_attention_kernels_over_scattered_pages(dtype, heads, kv_heads, dim, vdim, window, rot_dims):
    """A prompt of 150 tokens, then 60 single tokens, over pages 6, 1, 4, 0 of a pool; against the plain mixer with an identity as
    its output projection."""
    torch.manual_seed(heads * 100 + dim)
    width, eps, total = 48, 1e-5, 210
    mixer = bm.attention(heads, kv_heads, dim, vdim, window, rot_dims, base=300.0, diff=0.35)["mixer"]
    round_to = (lambda t: t.to(TORCH[dtype]).float())
    W = {"m.q": torch.randn(heads * 2 * dim, width) / 7, "m.k": torch.randn(kv_heads * 2 * dim, width) / 7, "m.v": torch.randn(kv_heads * vdim, width) / 7,
         "m.g": torch.randn(heads * vdim, width) / 7, "m.o": torch.eye(heads * vdim), "m.q.norm": 1 + 0.2 * torch.randn(dim), "m.k.norm": 1 + 0.2 * torch.randn(dim),
         "m.lq1": 0.3 * torch.randn(dim), "m.lk1": 0.3 * torch.randn(dim), "m.lq2": 0.3 * torch.randn(dim), "m.lk2": 0.3 * torch.randn(dim)}
    h = torch.randn(total, width)
    wanted = plain.differential_attention(h.double(), {name: value.double() for name, value in W.items()}, "m", mixer, eps)
    rows = attention_cache(mixer, 8, dtype, float("nan"))
    page_of = [6, 1, 4, 0]
    found = [run_attention_kernels(h[:150], W, mixer, eps, dtype, list(range(150)), page_of, rows)]
    for position in range(150, total):
        found.append(run_attention_kernels(h[position : position + 1], W, mixer, eps, dtype, [position], page_of, rows))
    assert relative_error(torch.cat(found), wanted) < (2e-5 if dtype == "float32" else 3e-2)
    for pool in rows if isinstance(rows, tuple) else (rows,):
        assert torch.isnan(pool[[2, 3, 5, 7]].float()).all()              # nothing was written outside the sequence's pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("vdim", [24, 32])      # one row per position; ordinary heads
def test_one_key_that_stands_out_is_seen_at_the_window_edge_and_not_beyond(dtype, vdim):
    """Queries whose first map points exactly along one key far back: the key sits on the window's last visible position for some
    queries and one position further for others (also across a page border); scores of 64 against a spread of a few make that key
    the whole softmax if it is seen, so a window that is one position off changes the result altogether."""
    torch.manual_seed(9)
    heads, kv_heads, dim, window, width, eps, total = 2, 1, 16, 33, 2 * 2 * 16, 1e-5, 200
    mixer = bm.attention(heads, kv_heads, dim, vdim, window, 0, scale=4.0, diff=0.2)["mixer"]
    # The input is the query itself: W_q is the identity, W_k picks the first head's first map.
    W = {"m.q": torch.eye(heads * 2 * dim, width), "m.k": torch.zeros(kv_heads * 2 * dim, width), "m.v": torch.randn(kv_heads * vdim, width) / 5,
         "m.g": torch.zeros(heads * vdim, width), "m.o": torch.eye(heads * vdim), "m.q.norm": torch.ones(dim), "m.k.norm": torch.ones(dim),
         "m.lq1": torch.zeros(dim), "m.lk1": torch.zeros(dim), "m.lq2": torch.zeros(dim), "m.lk2": torch.zeros(dim)}
    W["m.k"][:dim, :dim] = torch.eye(dim)
    W["m.k"][dim:, dim : 2 * dim] = torch.eye(dim)
    h = torch.randn(total, width).to(torch.bfloat16).float()
    for query in (40, 70, 96, 97, 128, 150, 199):
        h[query, :dim] = h[query - window + 1, :dim]           # just inside: the oldest position the query sees
    for query in (50, 80, 95, 129, 160, 190):
        h[query, :dim] = h[query - window, :dim]               # just outside
    wanted = plain.differential_attention(h.double(), {name: value.double() for name, value in W.items()}, "m", mixer, eps)
    rows = attention_cache(mixer, 4, dtype, 0.0)
    whole = run_attention_kernels(h, W, mixer, eps, dtype, list(range(total)), [2, 0, 3, 1], rows)
    # bfloat16 rounds queries and keys: a score of 64 moves by a quarter, its weight with it; a lost or added key moves the result by 0.3 or more
    assert relative_error(whole, wanted) < (2e-5 if dtype == "float32" else 8e-2)
    rows = attention_cache(mixer, 4, dtype, 0.0)
    singly = [run_attention_kernels(h[:30], W, mixer, eps, dtype, list(range(30)), [2, 0, 3, 1], rows)]
    singly += [run_attention_kernels(h[p : p + 1], W, mixer, eps, dtype, [p], [2, 0, 3, 1], rows) for p in range(30, total)]
    assert relative_error(torch.cat(singly), wanted) < (2e-5 if dtype == "float32" else 8e-2)
    # The test would see a window that is one off: the plain statement itself moves by far more than the tolerance.
    wider = plain.differential_attention(h.double(), {name: value.double() for name, value in W.items()}, "m", {**mixer, "mask": {"size": window + 1}}, eps)
    assert relative_error(wider, wanted) > 0.3


# ---- whole models: cuttings, batches, reuse --------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "one_tap"])
def test_whole_prompts_single_tokens_and_the_first_positions(models, name, dtype):
    engine, cfg, values = engine_of(models, name, dtype)
    tokens = tokens_for(cfg, 200, 21)
    wanted = plain_logits(cfg, values, tokens)
    whole = run_whole(engine, tokens)
    assert close(whole, wanted, dtype)
    assert close(whole[:4], wanted[:4], dtype)               # the first tokens: zeros before the convolution, one key in the window
    assert close(run_whole(engine, tokens[:1]), wanted[:1], dtype)
    stepwise = run_tail_stepwise(engine, tokens, 199)                              # every token but the first alone, through the graphs
    assert close(stepwise, wanted[1:], dtype)
    if dtype == "float32":
        assert relative_error(stepwise, whole[1:]) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_portions_down_to_two_tokens_and_page_borders(models, name, dtype):
    engine, cfg, values = engine_of(models, name, dtype)
    tokens = tokens_for(cfg, 330, 22)
    wanted = plain_logits(cfg, values, tokens)
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
@pytest.mark.parametrize("name", ["peaky", "edgy"])
def test_a_sharp_softmax_loses_no_key_far_back_at_a_page_border_or_at_the_window_edge(models, name, dtype):
    engine, cfg, values = engine_of(models, name, dtype)
    tokens = tokens_for(cfg, 400, 23)
    wanted = plain_logits(cfg, values, tokens)
    assert close(run_whole(engine, tokens), wanted, dtype)
    tail = run_tail_stepwise(engine, tokens, 150)                                  # decoded queries cross the borders at 256 and 320
    assert close(tail, wanted[-150:], dtype)
    slot = engine.open_sequence()                                                  # portions whose windows reach into earlier portions
    found = [engine.step([StepEntry(slot, tokens[begin : begin + 50], list(range(50)))]).float().cpu().clone() for begin in range(0, 400, 50)]
    engine.close_sequence(slot)
    assert close(torch.cat(found), wanted, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "edgy"])
def test_unequal_batches_against_each_request_alone(models, name, dtype):
    engine, cfg, values = engine_of(models, name, dtype, 2048)
    lengths, prompts = [90, 31, 140, 5, 66], [70, 1, 129, 3, 64]
    requests = [tokens_for(cfg, length, 30 + index) for index, length in enumerate(lengths)]
    together = run_batched(engine, requests, prompts)
    for request, prompt, rows in zip(requests, prompts, together):
        wanted = plain_logits(cfg, values, request)[prompt - 1 :]
        assert close(rows, wanted, dtype)
    engine.cache.check()
    assert engine.cache.slots.in_use == 0


def test_slots_pages_and_tails_that_are_used_again_start_clean(models):
    """A cache of three pages and as many slots: every request takes a slot whose convolution tail another left behind and pages
    that another wrote."""
    engine, cfg, values = engine_of(models, "mixed", "float32", 64 * 3)
    for round_number in range(4):
        requests = [tokens_for(cfg, length, 40 + 3 * round_number + index) for index, length in enumerate([60 + round_number, 40, 17])]
        together = run_batched(engine, requests, [len(request) - 6 for request in requests])
        for request, rows in zip(requests, together):
            assert relative_error(rows, plain_logits(cfg, values, request)[len(request) - 7 :]) < TOLERANCE["float32"]
        engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_sequence_in_a_cache_of_four_pages(models, dtype):
    """600 tokens through a cache that holds 256 positions: every layer has a window, so pages that fall out of it are given back
    and taken again; in runs and single tokens against the plain statement of the whole sequence."""
    engine, cfg, values = engine_of(models, "edgy", dtype, 64 * 4)
    tokens = tokens_for(cfg, 600, 25)
    wanted = plain_logits(cfg, values, tokens)
    slot = engine.open_sequence()
    found, position = [], 0
    for count in [50, 1, 1, 64, 30, 1, 1, 1, 50, 50, 50, 64, 1, 50, 50, 50, 36] + [1] * 50:
        piece = tokens[position : position + count]
        found.append(engine.step([StepEntry(slot, piece, list(range(len(piece))))]).float().cpu().clone())
        position += len(piece)
        engine.cache.check()
        assert all(len(group.held[slot]) <= 3 for group in engine.cache.kv.values())
    assert position == 600
    engine.close_sequence(slot)
    assert close(torch.cat(found), wanted, dtype)


def test_long_decoding_in_bfloat16_stays_with_the_plain_statement(models):
    engine, cfg, values = engine_of(models, "mixed", "bfloat16")
    tokens = tokens_for(cfg, 420, 24)
    wanted = plain_logits(cfg, values, tokens)
    assert close(run_tail_stepwise(engine, tokens, 400), wanted[-400:], "bfloat16")


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_greedy_generation_through_the_library_entry_point(models, name):
    folder, cfg, values = models[name]
    prompts = [tokens_for(cfg, length, 60 + index) for index, length in enumerate([9, 30, 2])]
    output = generate(folder, prompts, max_new_tokens=12, dtype="float32", stop_tokens=[])
    for prompt, result in zip(prompts, output):
        tokens = list(prompt)
        for _ in range(12):
            logits = plain_logits(cfg, values, tokens)[-1]
            best, second = torch.topk(logits, 2).values
            if float(best - second) < 1e-3 * float(logits.abs().max()):
                break                                                                # a close call proves nothing either way
            tokens.append(int(torch.argmax(logits)))
        made = len(tokens) - len(prompt)
        assert list(result.tokens[:made]) == tokens[len(prompt) :] and made >= 1


def test_trace_replay_of_a_bisudra_folder(models, tmp_path):
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
    wanted_a, wanted_b = plain_logits(cfg, values, first), plain_logits(cfg, values, second)
    rows = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, cfg["vocab"])
    assert relative_error(torch.from_numpy(rows), torch.stack([wanted_a[0], wanted_a[65], wanted_b[29]])) < TOLERANCE["float32"]
    rows = np.fromfile(out / "3.f32", dtype="<f4").reshape(2, cfg["vocab"])
    assert relative_error(torch.from_numpy(rows), torch.stack([wanted_a[68], wanted_b[32]])) < TOLERANCE["float32"]
    assert not (out / "4.f32").exists()


def test_the_command_line_on_a_bisudra_folder(models, tmp_path):
    """`bin/tau` on a Bisudra folder: greedy tokens in 32-bit equal those of `generate()`, with graphs and without, in chunks of
    prompt tokens; bfloat16 runs from the same folder; random weights are written for a Bisudra config.json and read back."""
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
    config_path.write_text(json.dumps(bm.PEAKY))
    drawn = str(tmp_path / "drawn")
    records = run(["--random-weights", str(config_path), "--model", drawn, "--seed", "4", "--max-tokens", "5", "--stop-ids", "", "--prompt-ids", "1,2,3"])
    assert [len(record["tokens"]) for record in records if "tokens" in record] == [5]
