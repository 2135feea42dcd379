"""The Tepavik decoder in the engine against the plain statement of ``tepavik_plain``.

Small configurations of their own, random weights, every position of every
request compared.  The scenarios run twice: on the CPU through the plain
statements of the kernels (``kernel_references.emulate_kernels``: what is under
test then is the configuration, the weights' names, the cache plan, state slots,
batch packing, replay and scheduler), and, marked ``gpu``, on the kernels in
float32 and bfloat16.
"""
from __future__ import annotations

import json
import math

import numpy as np
import pytest
import torch
from safetensors.torch import save_file

import tepavik_plain
import trace_tools
from conftest import random_tokens
from kernel_references import emulate_kernels


def attention(heads, kv_heads, dim, vdim, size, scale=0.4, softcap=6.0, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
             "mask": {"size": size}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer}


def lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}}


def mamba2(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def model(width, vocab, layers, ff, eps=1e-5):
    out = []
    for index, layer in enumerate(layers):
        layer = dict(layer)
        layer["mlp"] = None if ff[index] is None else {"kind": "dense", "ff": ff[index]}
        out.append(layer)
    return {"architecture": "Tepavik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": out}


CONFIGS = {
    # every mixer, key and value sizes that differ, a layer without a feed-forward, shared keys
    "mix": model(48, 97, [
        attention(4, 2, 16, 24, 7),
        lightning(3, 24, 16, [0.9, 0.999, 0.5]),
        mamba2(4, 12, 8, 2, 3, 2),
        attention(4, 2, 16, 24, 5, scale=0.7, softcap=3.0, kv_from=0),
        mamba2(6, 8, 20, 3, 5, 1),
    ], [64, 40, None, 56, 72]),
    # values the sizes above make unequal, here equal or 1: one key/value head, one group, one
    # norm part, a convolution of two taps, a chunk of one position, as many key/value heads as heads
    "ones": model(40, 61, [
        mamba2(2, 20, 16, 1, 2, 1),
        attention(2, 1, 24, 8, 1),
        lightning(1, 40, 8, [0.97]),
        attention(3, 3, 8, 40, 64, softcap=30.0),
        attention(3, 3, 8, 40, 3, kv_from=3),
    ], [48, None, 32, 32, 24], eps=1e-6),
    # head sizes the tensor-core attention kernels take, chunks that are no multiple of a page
    "wide": model(64, 83, [
        attention(4, 2, 64, 64, 50),
        lightning(2, 64, 64, [0.95, 0.999]),
        mamba2(4, 32, 64, 1, 4, 1),
        attention(4, 2, 64, 64, 33, scale=0.3, softcap=8.0, kv_from=0),
    ], [96, 96, 96, None]),
}
PAGE = {"mix": 4, "ones": 8, "wide": 16}
SINGLE = {
    "attention": model(32, 50, [attention(4, 2, 8, 16, 6)], [None]),
    "lightning": model(32, 50, [lightning(2, 16, 24, [0.8, 0.995])], [None]),
    "mamba2": model(32, 50, [mamba2(4, 8, 16, 2, 4, 2)], [None]),
    "mlp": model(32, 50, [lightning(1, 8, 8, [0.5])], [80]),
}


def write_folder(folder, config, seed):
    folder.mkdir(parents=True, exist_ok=True)
    weights = tepavik_plain.random_model(config, seed)
    (folder / "config.json").write_text(json.dumps(config))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return weights


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("tepavik")
    made = {}
    for index, (name, config) in enumerate({**CONFIGS, **SINGLE}.items()):
        made[name] = (base / name, config, write_folder(base / name, config, 10 + index))
    return made


def expected_rows(config, weights, requests):
    out = {}
    for name, tokens in requests.items():
        logits, _ = tepavik_plain.forward(config, weights, tokens)
        for position in range(len(tokens)):
            out[(name, position)] = logits[position].float().numpy()
    return out


def make_requests(config, lengths, seed=0):
    return {f"r{i}": random_tokens(config["vocab"], n, seed * 100 + i) for i, n in enumerate(lengths)}


def check(rows, expected, dtype):
    if dtype == "float32":
        trace_tools.compare(rows, expected, rtol=1e-4, atol=3e-5)
        return
    # bfloat16: the error of a row (mean taken off, root mean square) against the size of the logits
    assert set(rows) == set(expected)
    size = math.sqrt(float(np.mean([np.var(v) for v in expected.values()])))
    for key in sorted(expected):
        difference = rows[key] - expected[key]
        error = float(np.sqrt(np.mean((difference - difference.mean()) ** 2))) / size
        assert np.isfinite(rows[key]).all() and error < 0.04, f"first wrong token: {key}, error {error:.3f}"


def replay_modes(folder, config, weights, page, dtype, device, lengths=(1, 5, 9, 23, 37, 50)):
    from einf_b200.engine.replay import TraceReplayer

    requests = make_requests(config, lengths)
    expected = expected_rows(config, weights, requests)
    mixed_steps, most = trace_tools.mixed(requests, seed=3, page_round=page)
    room = -(-max(lengths) // 64) * 64
    traces = {
        "whole": (trace_tools.whole(requests), room),
        "tail": (trace_tools.last_one_by_one(requests, tail=12), room),
        "portions": (trace_tools.in_portions(requests), room),
        "mixed": (mixed_steps, most),
    }
    for mode, (steps, max_tokens) in traces.items():
        replayer = TraceReplayer(folder, dtype, max_tokens, block_len=page, device=device, max_requests=4)
        rows = trace_tools.run_steps(replayer, steps)
        check(rows, expected, dtype)
        assert replayer.manager.free_pages(0) == replayer.manager.group(0).num_pages, mode
        replayer.manager.check_invariants()


# ---------------------------------------------------------------------------
# the configuration and the weights' names
def test_configuration_names_every_tensor_of_the_design(folders):
    from einf_b200.config import TepavikConfig, load_config
    from einf_b200.parts.model import expected_tensors

    for name, (folder, config, weights) in folders.items():
        loaded = load_config(folder)
        assert isinstance(loaded, TepavikConfig)
        expected, optional = expected_tensors(loaded.model_spec())
        assert set(expected) == set(weights) and not optional, name
        for key, spec in expected.items():
            assert tuple(spec.shape) == tuple(weights[key].shape), key
    spec = load_config(folders["mix"][0]).model_spec()
    assert [entry.cache_from for entry in spec.schedule] == [None, None, None, 0, None]
    assert [layer.block for layer in spec.layers] == ["prenorm", "prenorm", "prenorm_mixer", "prenorm", "prenorm"]


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
    broken(lambda d: d["layers"][3]["mixer"].update(kv_from=3))          # not an earlier layer
    broken(lambda d: d["layers"][3]["mixer"].update(kv_from=1))          # not an attention layer
    broken(lambda d: d["layers"][1]["mixer"].update(decay=[0.5]))        # one decay per head
    broken(lambda d: d["layers"][2]["mixer"].update(groups=3))           # heads not a multiple
    broken(lambda d: d["layers"][0]["mlp"].update(kind="gated"))
    broken(lambda d: d["layers"][0]["mixer"].pop("scale"))
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
    assert set(tensors) == set(expected)
    step = torch.nn.functional.softplus(tensors["l0.mix.dt_bias"].float())
    assert 5e-4 < float(step.min()) and float(step.max()) < 0.2
    assert float(tensors["l0.norm1"].float().abs().max()) < 0.5      # stored around zero


def test_long_portions_are_cut_into_segments_only_where_that_fills_the_gpu():
    from einf_b200 import ops

    plan = ops.recurrence_plan
    assert plan(8, 1, 14, 64, 64, sms=148) == (1, 1)                 # decoding: the streaming kernel
    assert plan(4, 100, 14, 64, 64, sms=148) == (1, 100)             # short portions: one pass
    assert plan(1, 2048, 14, 64, 64, sms=148) == (16, 128)           # one prompt: sixteen segments
    assert plan(64, 2048, 32, 128, 128, sms=148) == (1, 2048)        # requests and heads fill the GPU already
    segments, length = plan(1, 100_000, 14, 64, 64, sms=148)         # at most 64 segments, whole tokens in all
    assert segments <= ops.MAX_SEGMENTS and segments * length >= 100_000 and length % 16 == 0
    segments, length = plan(4000, 300, 2, 16, 16, sms=148)           # requests x segments stay within the grid
    assert 4000 * segments <= 65535 and segments * length >= 300


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
        logits, _ = tepavik_plain.forward(config, weights, tokens)
        tokens.append(int(torch.argmax(logits[-1])))
    return tokens[len(prompt):]


def generation(folder, config, weights, dtype, device, lookahead=1, graphs=False):
    from einf_b200.config.engine import EngineConfig
    from einf_b200.engine import Engine

    prompts = [random_tokens(config["vocab"], n, 50 + n) for n in (3, 11, 1, 17, 6, 9)]
    engine = Engine.from_folder(folder, EngineConfig(
        dtype=dtype, block_len=4, num_blocks=48, max_batch_len=16, max_prefill_chunk_len=5, max_requests=4,
        device=device, use_cuda_graphs=graphs, decode_lookahead=lookahead))
    got = engine.generate(prompts, 8)
    assert engine.runner.num_state_slots == 4         # six requests through four slots: slots are used again
    return prompts, got


def test_greedy_generation_through_the_entry_point_emulated(folders, emulated):
    folder, config, weights = folders["mix"]
    prompts, got = generation(folder, config, weights, "float32", "cpu")
    for prompt, tokens in zip(prompts, got):
        assert tokens == greedy_plain(config, weights, prompt, 8)


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
# keys that decide a row.  Without positions a token's key and value depend on the token alone, so
# the weights are made for it: queries are the negated keys (no bias), which makes a token its own
# worst match, and token 1's embedding is the negative of token 0's, which makes token 1 (the
# needle) the best match of token 0 (the asker) while their values differ.  A needle stands early
# in every chunk; an asker at the chunk's last position sees it, the asker that opens the next
# chunk must see nothing but itself.
def needle_model(size):
    config = model(32, 40, [attention(2, 1, 16, 16, size, scale=1.5, softcap=40.0)], [None])
    weights = tepavik_plain.random_model(config, 5)
    weights["l0.mix.q"] = torch.cat([-weights["l0.mix.k"], -weights["l0.mix.k"]])
    for name in ("q.b", "k.b"):
        weights["l0.mix." + name] = torch.zeros_like(weights["l0.mix." + name])
    weights["embed"][1] = -weights["embed"][0]
    return config, weights


def needle_tokens(size, chunks):
    tokens = [2 + (i * 7) % 37 for i in range(size * chunks + 2)]
    for c in range(chunks):
        tokens[c * size + 1] = 1             # the needle, early in the chunk
        tokens[(c + 1) * size - 1] = 0       # the chunk's last position asks for it
        tokens[(c + 1) * size] = 0           # ... and so does the first of the next, which has only itself
    return tokens


def needle_check(tmp_path, dtype, device, size=24, page=16):
    from einf_b200.engine.replay import TraceReplayer

    config, weights = needle_model(size)
    folder = tmp_path / "needle"
    folder.mkdir(exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    requests = {"n": needle_tokens(size, 3)}
    expected = expected_rows(config, weights, requests)
    # the plain statement itself must feel the edge: one position on, the needle is out of sight
    inside, outside = expected[("n", 2 * size - 1)], expected[("n", 2 * size)]
    assert np.abs(inside - outside).max() > 0.5
    for steps in (trace_tools.whole(requests), trace_tools.last_one_by_one(requests, tail=size + 3),
                  trace_tools.in_portions(requests, sizes=(size - 1, 2, size, 3))):
        replayer = TraceReplayer(folder, dtype, 128, block_len=page, device=device)
        check(trace_tools.run_steps(replayer, steps), expected, dtype)


def test_a_key_at_a_chunks_edge_decides_the_row_emulated(tmp_path, emulated):
    needle_check(tmp_path, "float32", "cpu")


# ---------------------------------------------------------------------------
# the kernels (GPU)
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(name, dtype, folders):
    folder, config, weights = folders[name]
    replay_modes(folder, config, weights, 4, dtype, "cuda:0", lengths=(1, 6, 19, 70))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_replay_modes(name, dtype, folders):
    folder, config, weights = folders[name]
    replay_modes(folder, config, weights, PAGE[name], dtype, "cuda:0", lengths=(1, 5, 9, 23, 37, 50, 131))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_at_a_chunks_edge_decides_the_row(dtype, tmp_path):
    needle_check(tmp_path, dtype, "cuda:0")


@pytest.mark.gpu
def test_long_decoding_keeps_the_state(folders):
    """Three hundred tokens one by one after a short prompt: the recurrent states and the
    convolution's inputs are carried from step to step, the chunks' edges pass many times."""
    from einf_b200.engine.replay import TraceReplayer

    folder, config, weights = folders["mix"]
    requests = make_requests(config, [310], seed=7)
    expected = expected_rows(config, weights, requests)
    replayer = TraceReplayer(folder, "float32", 320, block_len=PAGE["mix"], device="cuda:0")
    rows = trace_tools.run_steps(replayer, trace_tools.last_one_by_one(requests, tail=300))
    check(rows, expected, "float32")


@pytest.mark.gpu
@pytest.mark.parametrize("lookahead,graphs", [(1, False), (1, True), (4, True)])
def test_greedy_generation_through_the_entry_point(lookahead, graphs, folders):
    folder, config, weights = folders["mix"]
    prompts, got = generation(folder, config, weights, "float32", "cuda:0", lookahead, graphs)
    for prompt, tokens in zip(prompts, got):
        assert tokens == greedy_plain(config, weights, prompt, 8)
