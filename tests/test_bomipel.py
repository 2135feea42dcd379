"""The Bomipel decoder in the engine against the plain statement of ``bomipel_plain``.

Small configurations of their own, random weights, every position of every request compared.
The scenarios run twice: on the CPU through the plain statements of the kernels
(``kernel_references.emulate_kernels``: what is under test then is the configuration, the weights'
names, the cache plan with its windowed groups, batch packing, replay and scheduler), and, marked
``gpu``, on the kernels in float32 and bfloat16.

A routed feed-forward makes bfloat16 comparisons delicate: where two router logits are closer than
the rounding of the router's input, either expert may be taken, and everything after that token
differs; with a few routed layers that happens within a dozen tokens.  So the bfloat16 scenarios run
a variant of every configuration in which each token takes all experts of a layer (the same weights,
``top`` = ``experts``: every kernel of the routed path runs, no choice can flip) and compare every
position; which experts are chosen is float32's to test, and the router kernel's own test.
"""
from __future__ import annotations

import json
import math
import random

import numpy as np
import pytest
import torch
from safetensors.torch import save_file

import bomipel_plain
import trace_tools
from conftest import random_tokens
from kernel_references import emulate_kernels

SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}


def attention(heads, kv_heads, dim, vdim, size=None, keep_first=0, rot_dims=None, base=10000.0, scaling=None,
              v_mix=False, scale=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
             "scale": scale if scale is not None else dim ** -0.5}
    if size is not None:
        mixer["mask"] = {"size": size, "keep_first": keep_first}
    if rot_dims:
        mixer["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            mixer["rot"]["scaling"] = scaling
    if v_mix:
        mixer["v_mix"] = True
    return {"type": "attention", "mixer": mixer}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, base=10000.0, scale=None):
    return {"type": "latent_attention", "mixer": {
        "heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
        "rot": {"base": base, "dims": rot_dim}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def model(width, vocab, layers, mlps, eps=1e-5, softcap=12.0):
    out = []
    for layer, mlp in zip(layers, mlps):
        layer = dict(layer)
        layer["mlp"] = mlp
        out.append(layer)
    config = {"architecture": "Bomipel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": out}
    if softcap is not None:
        config["logit_softcap"] = softcap
    return config


CONFIGS = {
    # both mixers, windows of two sizes (two page groups), partial rotation with scaling, three
    # value-mixing layers, a layer without a feed-forward, two of four and three of five experts
    "mix": model(48, 97, [
        attention(4, 2, 16, 24, size=9, keep_first=3, rot_dims=8, scaling=SCALING, v_mix=True),
        latent(3, 16, 8, 12, 24, 20),
        attention(6, 2, 8, 24, size=21, keep_first=5, rot_dims=8, base=500.0, v_mix=True),
        attention(2, 2, 24, 24, size=9, keep_first=3, rot_dims=16, v_mix=True),
        latent(2, 8, 16, 24, 16, 40, base=300.0),
    ], [moe(40, 4, 2), moe(24, 5, 3), None, moe(56, 3, 1), moe(32, 4, 2)]),
    # values the sizes above make unequal, here equal or 1: one key/value head and as many as heads, a
    # window of one key, nothing kept, every dimension rotated, one expert of one, all experts chosen,
    # a layer without a mask, no cap on the logits
    "ones": model(40, 61, [
        attention(2, 1, 8, 8, size=1, keep_first=0, rot_dims=8),
        attention(3, 3, 16, 8, size=4, keep_first=4, rot_dims=2, v_mix=True),
        latent(1, 8, 2, 8, 8, 8),
        attention(2, 2, 8, 16, rot_dims=4, scaling={"factor": 2.0, "low": 1.0, "high": 2.0, "original": 16}),
        attention(3, 3, 24, 8, size=64, keep_first=1, v_mix=True),
    ], [moe(16, 1, 1), moe(24, 3, 3), None, moe(8, 2, 1), moe(16, 6, 1)], eps=1e-6, softcap=None),
    # larger heads, windows that are no multiple of a page, a latent row of 80
    "wide": model(64, 83, [
        latent(4, 32, 16, 32, 64, 48),
        attention(4, 2, 64, 32, size=50, keep_first=17, rot_dims=32, scaling=SCALING, v_mix=True),
        attention(6, 2, 32, 32, size=33, keep_first=2, rot_dims=32, v_mix=True),
    ], [moe(96, 8, 2), moe(64, 4, 1), moe(32, 16, 4)]),
    # sizes the tensor-core kernels take: latent rows of 128 and 64, windowed layers with heads of 64,
    # nothing kept, a few positions kept, more positions kept than the window is wide
    "cores": model(64, 83, [
        latent(4, 32, 32, 32, 96, 48),
        attention(4, 2, 64, 64, size=40, keep_first=0, rot_dims=32),
        latent(2, 16, 16, 24, 48, 32, base=700.0),
        attention(2, 1, 64, 64, size=21, keep_first=5, rot_dims=16, v_mix=True),
        attention(2, 1, 128, 64, size=33, keep_first=3, v_mix=True),
        attention(3, 1, 64, 64, size=19, keep_first=70, rot_dims=64, v_mix=True),
    ], [moe(64, 4, 2), moe(32, 2, 1), None, moe(48, 3, 2), None, moe(32, 2, 2)]),
}
PAGE = {"mix": 4, "ones": 8, "wide": 16, "cores": 16}
SINGLE = {
    "attention": model(32, 50, [attention(4, 2, 8, 16, size=6, keep_first=2, rot_dims=4)], [None]),
    "latent": model(32, 50, [latent(2, 8, 4, 12, 16, 24)], [None]),
    "routed": model(32, 50, [attention(1, 1, 8, 8, rot_dims=8)], [moe(24, 6, 2)]),
    "value_mix": model(32, 50, [attention(2, 1, 8, 12, rot_dims=8, v_mix=True), latent(2, 8, 4, 12, 16, 24),
                                attention(4, 1, 16, 12, rot_dims=8, v_mix=True)], [None, None, None]),
}


def write_folder(folder, config, weights):
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))


def all_experts(config):
    """The same model with every expert of a layer chosen for every token."""
    config = json.loads(json.dumps(config))
    for layer in config["layers"]:
        if layer["mlp"] is not None:
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return config


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("bomipel")
    made = {}
    for index, (name, config) in enumerate({**CONFIGS, **SINGLE}.items()):
        weights = bomipel_plain.random_model(config, 20 + index)
        write_folder(base / name, config, weights)
        made[name] = (base / name, config, weights)
        write_folder(base / (name + "_all"), all_experts(config), weights)
        made[name + "_all"] = (base / (name + "_all"), all_experts(config), weights)
    return made


def expected_rows(config, weights, requests):
    """Logits of every position, and per request the first position whose router choice is a close call."""
    out, close = {}, {}
    for name, tokens in requests.items():
        margins = []
        logits, _ = bomipel_plain.forward(config, weights, tokens, margins=margins)
        for position in range(len(tokens)):
            out[(name, position)] = logits[position].float().numpy()
        close[name] = len(tokens)
        if margins:
            tight = (torch.stack(margins).min(0).values < 0.25).nonzero()
            if len(tight):
                close[name] = int(tight[0])
    return out, close


def make_requests(config, lengths, seed=0):
    return {f"r{i}": random_tokens(config["vocab"], n, seed * 100 + i) for i, n in enumerate(lengths)}


def check(rows, expected, dtype, close=None):
    if dtype == "float32":
        trace_tools.compare(rows, expected, rtol=1e-4, atol=3e-5)
        return 0
    # bfloat16: the error of a row (mean taken off, root mean square) against the size of the logits
    assert set(rows) == set(expected)
    size = math.sqrt(float(np.mean([np.var(v) for v in expected.values()])))
    compared = 0
    for key in sorted(expected):
        assert np.isfinite(rows[key]).all()
        if close is not None and key[1] >= close[key[0]]:
            continue
        difference = rows[key] - expected[key]
        error = float(np.sqrt(np.mean((difference - difference.mean()) ** 2))) / size
        assert error < 0.03, f"first wrong token: {key}, error {error:.3f}"
        compared += 1
    assert compared == len(expected) or close is not None
    return compared


def replay_modes(folder, config, weights, page, dtype, device, lengths=(1, 5, 9, 23, 37, 50)):
    from einf_b200.engine.replay import TraceReplayer

    requests = make_requests(config, lengths)
    expected, close = expected_rows(config, weights, requests)
    mixed_steps, most = trace_tools.mixed(requests, seed=3, page_round=page)
    room = -(-max(lengths) // 64) * 64
    traces = {
        "whole": (trace_tools.whole(requests), room),
        "tail": (trace_tools.last_one_by_one(requests, tail=30), room),
        "portions": (trace_tools.in_portions(requests), room),
        "mixed": (mixed_steps, most),
    }
    for mode, (steps, max_tokens) in traces.items():
        replayer = TraceReplayer(folder, dtype, max_tokens, block_len=page, device=device, max_requests=4)
        rows = trace_tools.run_steps(replayer, steps)
        check(rows, expected, dtype, close)
        manager = replayer.manager
        for group in range(manager.num_groups):     # every page of every group came back
            assert manager.free_pages(group) == manager.group(group).num_pages, (mode, group)
        manager.check_invariants()


# ---------------------------------------------------------------------------
# the configuration and the weights' names
def test_configuration_names_every_tensor_of_the_design(folders):
    from einf_b200.config import BomipelConfig, load_config
    from einf_b200.parts.model import expected_tensors

    for name, (folder, config, weights) in folders.items():
        loaded = load_config(folder)
        assert isinstance(loaded, BomipelConfig)
        expected, optional = expected_tensors(loaded.model_spec())
        assert set(expected) == set(weights), name
        for key, spec in expected.items():
            assert tuple(spec.shape) == tuple(weights[key].shape), key
    spec = load_config(folders["mix"][0]).model_spec()
    assert [layer.block for layer in spec.layers] == ["parallel", "parallel", "prenorm_mixer", "parallel", "parallel"]
    assert [layer.parts["mixer"].get("value_mix") for layer in spec.layers] == ["source", None, "blend", "blend", None]
    assert spec.head["tied_to"] == "embed" and spec.head["softcap"] == 12.0


def test_windows_that_keep_first_positions_are_page_groups_of_their_own(folders, emulated):
    from einf_b200.config.engine import EngineConfig
    from einf_b200.engine.runner import ModelRunner

    folder, config, weights = folders["mix"]
    runner = ModelRunner.from_folder(folder, EngineConfig(
        dtype="float32", block_len=4, num_blocks=64, max_batch_len=16, max_prefill_chunk_len=16, max_requests=2,
        device="cpu", use_cuda_graphs=False))
    plan = runner.model.cache_plan
    # layers 0 and 3 share (9, 3); layer 2 has (21, 5); the latent layers keep everything
    assert sorted(zip(plan.group_windows, plan.group_keeps), key=str) == sorted([(9, 3), (None, 0), (21, 5)], key=str)
    assert plan.entries[0].group == plan.entries[3].group != plan.entries[2].group
    assert plan.entries[1].need.value_size == 0 and plan.entries[1].need.head_size == 24 + 8
    assert [g.keep_first for g in runner.group_specs()] == list(plan.group_keeps)


def test_configuration_refuses_what_the_design_does_not_have():
    from einf_b200.config import ConfigError, config_from_dict

    good = CONFIGS["mix"]
    config_from_dict(good)

    def broken(change):
        data = json.loads(json.dumps(good))
        change(data)
        with pytest.raises(ConfigError):
            config_from_dict(data)

    broken(lambda d: d["layers"][0].update(type="conv"))
    broken(lambda d: d["layers"][0]["mixer"].update(kv_heads=3))            # heads not a multiple
    broken(lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7))         # odd
    broken(lambda d: d["layers"][0]["mixer"]["rot"].update(dims=32))        # more than the head has
    broken(lambda d: d["layers"][0]["mixer"]["rot"]["scaling"].pop("low"))
    broken(lambda d: d["layers"][0]["mixer"]["mask"].update(size=0))
    broken(lambda d: d["layers"][2]["mixer"].update(vdim=8))                # cannot be mixed with layer 0's values
    broken(lambda d: d["layers"][1]["mixer"]["rot"].update(dims=4))         # must be rot_dim
    broken(lambda d: d["layers"][1]["mixer"].pop("kv_rank"))
    broken(lambda d: d["layers"][0]["mlp"].update(kind="dense"))
    broken(lambda d: d["layers"][0]["mlp"]["router"].update(top=5))         # more than experts
    broken(lambda d: d.update(logit_softcap=0))
    broken(lambda d: d.pop("width"))
    broken(lambda d: d["norm"].update(eps=0))


def test_random_weights_mode_writes_a_folder_the_loader_takes(tmp_path):
    from einf_b200.config import config_from_dict, load_config
    from einf_b200.parts.model import expected_tensors
    from einf_b200.weights import load_tensors, write_random_model

    folder = write_random_model(tmp_path / "m", config_from_dict(CONFIGS["ones"]), seed=4)
    config = load_config(folder)
    expected, optional = expected_tensors(config.model_spec())
    tensors = load_tensors(folder, expected, optional=optional)
    assert set(tensors) == set(expected) == set(bomipel_plain.tensor_shapes(CONFIGS["ones"]))
    assert 0 < float(tensors["l1.mix.vmix"]) < 1 and tensors["l1.mix.vmix"].shape == ()


def test_frequency_scaling_keeps_short_wavelengths_and_stretches_long_ones():
    from einf_b200.parts.position import RotaryPosition

    table = RotaryPosition.scaled_frequencies(10000.0, 32, SCALING).double()
    plain = bomipel_plain.rotary_frequencies(10000.0, 32)
    want = bomipel_plain.rotary_frequencies(10000.0, 32, SCALING)
    assert torch.allclose(table, want, rtol=1e-6)
    ratio = (plain / want)
    assert ratio[0] == 1.0 and abs(float(ratio[-1]) - 8.0) < 1e-9          # the two ends
    assert ((ratio > 1.0 + 1e-9) & (ratio < 8.0 - 1e-9)).any()            # and a blended one between


# ---------------------------------------------------------------------------
# the engine on the plain statements of the kernels (CPU)
@pytest.fixture()
def emulated():
    with emulate_kernels():
        yield


@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone_emulated(name, folders, emulated):
    folder, config, weights = folders[name]
    replay_modes(folder, config, weights, 4, "float32", "cpu", lengths=(1, 6, 19))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_replay_modes_emulated(name, folders, emulated):
    folder, config, weights = folders[name]
    replay_modes(folder, config, weights, PAGE[name], "float32", "cpu")


def greedy_plain(config, weights, prompt, new):
    tokens = list(prompt)
    for _ in range(new):
        logits, _ = bomipel_plain.forward(config, weights, tokens)
        tokens.append(int(torch.argmax(logits[-1])))
    return tokens[len(prompt):]


def generation(folder, config, weights, dtype, device, lookahead=1, graphs=False):
    from einf_b200.config.engine import EngineConfig
    from einf_b200.engine import Engine

    prompts = [random_tokens(config["vocab"], n, 50 + n) for n in (3, 11, 1, 17, 6, 9)]
    engine = Engine.from_folder(folder, EngineConfig(
        dtype=dtype, block_len=4, num_blocks=48, max_batch_len=16, max_prefill_chunk_len=5, max_requests=4,
        device=device, use_cuda_graphs=graphs, decode_lookahead=lookahead))
    got = engine.generate(prompts, 14)       # past the smaller window: its pages go back while decoding
    return prompts, got


def test_greedy_generation_through_the_entry_point_emulated(folders, emulated):
    folder, config, weights = folders["mix"]
    prompts, got = generation(folder, config, weights, "float32", "cpu")
    for prompt, tokens in zip(prompts, got):
        assert tokens == greedy_plain(config, weights, prompt, 14)


def test_command_line_runs_the_design(folders, emulated, capsys, tmp_path):
    from einf_b200.cli.run_qwen import main

    folder, config, weights = folders["mix"]
    prompt = [5, 17, 3, 90, 4, 8, 2]
    code = main(["--model-dir", str(folder), "--prompt-ids", ",".join(map(str, prompt)), "--dtype", "float32",
                 "--max-new-len", "5", "--max-prefill-chunk-len", "3", "--block-len", "4", "--max-requests", "2",
                 "--device", "cpu", "--compare-reference"], prog="run_model")
    out = capsys.readouterr().out
    assert code == 0, out
    fields = dict(line.split(": ", 1) for line in out.splitlines() if ": " in line)
    assert json.loads(fields["generated_ids"]) == greedy_plain(config, weights, prompt, 5)
    assert fields["tokens_equal"] == "True" and fields["completion_reason"] == "length"
    # random weights from a bare config.json of the design
    path = tmp_path / "config.json"
    path.write_text(json.dumps(CONFIGS["ones"]))
    code = main(["--random-weights", "--config", str(path), "--seed", "3", "--prompt-ids", "7,8,9", "--dtype", "float32",
                 "--max-new-len", "4", "--block-len", "8", "--device", "cpu"])
    out = capsys.readouterr().out
    assert code == 0 and "generated_ids: [" in out, out


# ---------------------------------------------------------------------------
# Keys that decide a row.  With random weights a key among many moves a row by little, and an edge
# that is one position off hides in the tolerance.  So the weights are made for it: a query is the
# negated key of its token (no feed-forward, one layer), which makes a token its own worst match,
# and token 1's embedding is the negative of token 0's, which makes token 1 (the needle) the best
# match of token 0 (the asker) at any distance on the dimensions that are not rotated, while their
# values are opposite.  Whether an asker sees a needle then decides its logits.
def needle_attention(size, keep_first, kv_heads=1):
    config = model(32, 40, [attention(2, kv_heads, 16, 16, size=size, keep_first=keep_first, rot_dims=4, scale=1.2)],
                   [None], softcap=None)
    weights = bomipel_plain.random_model(config, 5)
    key = weights["l0.mix.k"]
    weights["l0.mix.q"] = torch.cat([-key] * (2 // kv_heads))
    weights["embed"][1] = -weights["embed"][0]
    return config, weights


def needle_latent():
    config = model(32, 40, [latent(2, 16, 4, 16, 24, 24, scale=1.2)], [None], softcap=None)
    weights = bomipel_plain.random_model(config, 6)
    # the query latent is the key/value latent; the plain part of a query is the negated plain key
    weights["l0.mix.dq"] = weights["l0.mix.dkv"][:24].clone()
    weights["l0.mix.dq.norm"] = weights["l0.mix.dkv.norm"].clone()
    up = weights["l0.mix.uq"].reshape(2, 20, 24).clone()
    up[:, :16] = -weights["l0.mix.uk"].reshape(2, 16, 24)
    up[:, 16:] *= 0.1
    weights["l0.mix.uq"] = up.reshape(40, 24)
    weights["embed"][1] = -weights["embed"][0]
    return config, weights


def run_needle(tmp_path, config, weights, tokens, pairs, dtype, device, page, tail, portions):
    """``pairs``: (position that sees a needle, position of the same kind that must not)."""
    from einf_b200.engine.replay import TraceReplayer

    folder = tmp_path / "needle"
    write_folder(folder, config, weights)
    requests = {"n": tokens}
    expected, _ = expected_rows(config, weights, requests)
    for inside, outside in pairs:      # the plain statement itself must feel the edge
        assert np.abs(expected[("n", inside)] - expected[("n", outside)]).max() > 0.5, (inside, outside)
    room = -(-len(tokens) // 64) * 64
    for steps in (trace_tools.whole(requests), trace_tools.last_one_by_one(requests, tail=tail),
                  trace_tools.in_portions(requests, sizes=portions)):
        replayer = TraceReplayer(folder, dtype, room, block_len=page, device=device)
        check(trace_tools.run_steps(replayer, steps), expected, dtype)


def window_needle(tmp_path, dtype, device, size=24, keep=3, page=16):
    """Askers (token 0) and needles (token 1) around every edge: a needle ``size - 1`` back is the last
    one seen, ``size`` back the first one lost; a needle at position ``keep - 1`` is seen from
    anywhere, one at ``keep`` only from within the window."""
    config, weights = needle_attention(size, keep)
    length = 4 * size + 9
    tokens = [2 + (i * 7) % 37 for i in range(length)]
    tokens[keep - 1] = 1                       # kept for good
    first_in = 2 * size + 5                    # far beyond the window, sees only the kept needle
    tokens[first_in] = 0
    config_out, weights_out = config, weights
    # window edge: needle at p, askers at p + size - 1 (sees it) and, in a second sequence, p + size
    p = size + 7
    inside, outside = list(tokens), list(tokens)
    inside[keep - 1] = outside[keep - 1] = 5   # no kept needle in these two
    inside[p] = outside[p] = 1
    inside[p + size - 1] = 0
    outside[p + size] = 0
    run_needle(tmp_path / "kept", config, weights, tokens, [], dtype, device, page, size + 9, (size - 1, 2, size, 3))
    # the kept needle at keep - 1 is seen, the same needle at keep is not
    moved = list(tokens)
    moved[keep - 1], moved[keep] = 5, 1
    folder_rows = {}
    for name, sequence in (("kept", tokens), ("moved", moved), ("inside", inside), ("outside", outside)):
        logits, _ = bomipel_plain.forward(config, weights, sequence)
        folder_rows[name] = logits.float().numpy()
    assert np.abs(folder_rows["kept"][first_in] - folder_rows["moved"][first_in]).max() > 0.5
    assert np.abs(folder_rows["inside"][p + size - 1] - folder_rows["outside"][p + size]).max() > 0.5
    for name, sequence in (("moved", moved), ("inside", inside), ("outside", outside)):
        run_needle(tmp_path / name, config_out, weights_out, sequence, [], dtype, device, page, size + 9,
                   (size - 1, 2, size, 3))


def far_needle(tmp_path, dtype, device, page=16):
    """Latent attention sees everything: a needle at position 3 among three hundred keys, askers at a
    page's last and first slot and at the very end; a second asker-free position for contrast."""
    config, weights = needle_latent()
    tokens = [2 + (i * 11) % 37 for i in range(300)]
    tokens[3] = 1
    for asker in (8 * page - 1, 8 * page, 299):
        tokens[asker] = 0
    without = list(tokens)
    without[3] = 7
    with_rows = bomipel_plain.forward(config, weights, tokens)[0].float().numpy()
    without_rows = bomipel_plain.forward(config, weights, without)[0].float().numpy()
    assert np.abs(with_rows[299] - without_rows[299]).max() > 0.5
    run_needle(tmp_path / "far", config, weights, tokens, [], dtype, device, page, 40, (100, 2, 27, 64))


def test_keys_at_the_windows_edges_decide_the_rows_emulated(tmp_path, emulated):
    window_needle(tmp_path, "float32", "cpu")


def test_a_far_key_decides_the_row_emulated(tmp_path, emulated):
    far_needle(tmp_path, "float32", "cpu")


# ---------------------------------------------------------------------------
# seeded random configurations: sizes, head counts, layer order, windows and constants drawn anew
def random_config(rng):
    width, vocab = rng.choice([64, 96, 120, 192]), rng.choice([97, 512, 1000])
    layers, mlps, mixed_shape = [], [], None
    for _ in range(rng.randint(2, 5)):
        if rng.random() < 0.5:
            kv_heads = rng.choice([1, 2, 3])
            heads = kv_heads * rng.choice([1, 2, 4])
            dim, vdim = rng.choice([16, 24, 40, 56, 64, 128]), rng.choice([16, 24, 40, 64, 128])
            if rng.random() < 0.4:
                vdim = dim
            v_mix = rng.random() < 0.6
            if v_mix and mixed_shape is None:
                mixed_shape = (kv_heads, vdim)
            elif v_mix:
                kv_heads, vdim = mixed_shape
                heads = kv_heads * rng.choice([1, 2, 4])
            rot = rng.choice([None, 2, dim // 4 * 2, dim])
            scaling = rng.choice([None, {"factor": 8.0, "low": 1.0, "high": 2.0, "original": rng.choice([64, 2048])}])
            layers.append(attention(heads, kv_heads, dim, vdim, size=rng.choice([None, 1, 17, 64, 80, 200]),
                                    keep_first=rng.choice([0, 1, 5, 40, 150]), rot_dims=rot,
                                    base=rng.choice([500.0, 1e4, 3e5]), scaling=scaling if rot else None, v_mix=v_mix))
        else:
            rank, rot = rng.choice([(16, 8), (32, 32), (48, 16), (56, 8), (96, 32), (40, 24), (120, 8)])
            layers.append(latent(rng.choice([2, 4, 6]), rng.choice([16, 32, 64]), rot, rng.choice([16, 48, 64]), rank,
                                 rng.choice([24, 80]), base=rng.choice([300.0, 2e6])))
        experts = rng.choice([1, 2, 8, 16])
        mlps.append(None if rng.random() < 0.2 else moe(rng.choice([24, 72, 100]), experts, rng.randint(1, min(experts, 4))))
    return model(width, vocab, layers, mlps, eps=rng.choice([1e-5, 1e-6]), softcap=rng.choice([None, 20.0, 30.0]))


def row_errors(rows, expected):
    """Per row: the difference's root mean square (mean taken off) over the spread of the logits."""
    size = math.sqrt(float(np.mean([np.var(v) for v in expected.values()])))
    out = {}
    for key, want in expected.items():
        difference = rows[key] - want
        out[key] = float(np.sqrt(np.mean((difference - difference.mean()) ** 2))) / size
    return out


def random_configuration_check(seed, tmp_path, device, lengths, dtypes):
    from einf_b200.engine.replay import TraceReplayer

    config = random_config(random.Random(seed))
    weights = bomipel_plain.random_model(config, seed)
    for dtype in dtypes:
        used = config if dtype == "float32" else all_experts(config)
        folder = tmp_path / f"{seed}_{dtype}"
        write_folder(folder, used, weights)
        requests = make_requests(used, lengths, seed)
        expected, _ = expected_rows(used, weights, requests)
        mixed_steps, most = trace_tools.mixed(requests, seed=seed, page_round=64)
        room = -(-max(lengths) // 64) * 64
        for steps, tokens in ((trace_tools.whole(requests), room), (trace_tools.last_one_by_one(requests, tail=40), room),
                              (trace_tools.in_portions(requests, sizes=(100, 2, 64, 3, 29, 128)), room), (mixed_steps, most)):
            replayer = TraceReplayer(folder, dtype, tokens, device=device)
            errors = row_errors(trace_tools.run_steps(replayer, steps), expected)
            worst = max(errors, key=errors.get)
            # 32-bit: a long prompt's rounding stays thirty times below this; bfloat16 as in ``check``
            assert errors[worst] < (2.5e-5 if dtype == "float32" else 0.03), (seed, dtype, worst, errors[worst], config)
            replayer.manager.check_invariants()


@pytest.mark.parametrize("seed", [31, 32])
def test_random_configurations_emulated(seed, tmp_path, emulated):
    random_configuration_check(seed, tmp_path, "cpu", (1, 9, 40, 75), ("float32",))


# ---------------------------------------------------------------------------
# the kernels (GPU)
@pytest.mark.gpu
@pytest.mark.parametrize("seed", [1, 2, 3, 5, 9, 17, 18])
def test_random_configurations(seed, tmp_path):
    random_configuration_check(seed, tmp_path, "cuda:0", (1, 23, 97, 402, 1115) if seed % 2 else (2, 50, 330, 700),
                               ("float32", "bfloat16"))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(name, dtype, folders):
    folder, config, weights = folders[name if dtype == "float32" else name + "_all"]
    replay_modes(folder, config, weights, 4, dtype, "cuda:0", lengths=(1, 6, 19, 70))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_replay_modes(name, dtype, folders):
    folder, config, weights = folders[name if dtype == "float32" else name + "_all"]
    replay_modes(folder, config, weights, PAGE[name], dtype, "cuda:0", lengths=(1, 5, 9, 23, 37, 50, 131))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_at_the_windows_edges_decide_the_rows(dtype, tmp_path):
    window_needle(tmp_path, dtype, "cuda:0")
    window_needle(tmp_path / "page", dtype, "cuda:0", size=32, keep=16, page=16)   # edges on page borders


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_decides_the_row(dtype, tmp_path):
    far_needle(tmp_path, dtype, "cuda:0")


@pytest.mark.gpu
def test_long_decoding_passes_the_windows_many_times(folders):
    """Three hundred tokens one by one after a short prompt: the windows move on, their pages go back
    to the pool, the kept first pages stay."""
    from einf_b200.engine.replay import TraceReplayer

    folder, config, weights = folders["mix"]
    requests = make_requests(config, [310], seed=7)
    expected, _ = expected_rows(config, weights, requests)
    replayer = TraceReplayer(folder, "float32", 320, block_len=PAGE["mix"], device="cuda:0")
    rows = trace_tools.run_steps(replayer, trace_tools.last_one_by_one(requests, tail=300))
    check(rows, expected, "float32")


@pytest.mark.gpu
@pytest.mark.parametrize("lookahead,graphs", [(1, False), (1, True), (4, True)])
def test_greedy_generation_through_the_entry_point(lookahead, graphs, folders):
    folder, config, weights = folders["mix"]
    prompts, got = generation(folder, config, weights, "float32", "cuda:0", lookahead, graphs)
    for prompt, tokens in zip(prompts, got):
        assert tokens == greedy_plain(config, weights, prompt, 14)
