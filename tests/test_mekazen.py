"""The Mekazen decoder in the engine against the plain implementation
(``plain_mekazen.py``): its configuration and mechanisms one at a time, then
whole prompts, decoding through the cache, portions, mixed batches, pages that
come back, edges of chunks, the first tokens, generation through the
scheduler, the command line and the trace program. Every model here is tiny,
made for the test with random weights, and differs from layer to layer."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_mekazen as plain
import replay_helpers as cuts
from conftest import ROOT, random_ids


# ------------------------------------------------------------ configurations
def layer(heads, kv_heads, dim, chunk, rot, ff, scale):
    mixer = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": dim}
    if chunk:
        mixer["mask"] = {"size": chunk}
    if rot:
        mixer["rot"] = rot
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def bands(factor, low, high, original):
    return {"factor": factor, "low": low, "high": high, "original": original}


# SMALL: head sizes the vector paths do not take (12), a layer without a
# feed-forward, one key/value head for all query heads and one per query head,
# chunks below and above a page, one pair rotated and a whole head rotated,
# frequencies in all three bands of the stretch.
SMALL = {"architecture": "Mekazen", "vocab": 211, "width": 72, "norm": {"eps": 1e-6}, "logit_softcap": 4.0,
         "layers": [
             layer(4, 2, 16, 24, {"base": 1.0e4, "dims": 8, "scaling": bands(4.0, 0.5, 3.0, 40)}, 96, 0.3),
             layer(3, 3, 24, 40, {"base": 5.0e3, "dims": 24}, 0, 0.2),
             layer(6, 1, 12, 7, {"base": 1.0e2, "dims": 2, "scaling": bands(2.5, 2.0, 16.0, 100)}, 56, 0.35)]}
# WIDE: heads of 64 and 128 values (the tensor-core prompt kernels, the
# split-key decode kernel and its merge with the projection in bfloat16), a
# chunk that ends inside a page (50), one larger than a key tile (130), layers
# whose caches differ in shape.
WIDE = {"architecture": "Mekazen", "vocab": 300, "width": 128, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
        "layers": [
            layer(6, 2, 64, 50, {"base": 1.0e5, "dims": 32, "scaling": bands(8.0, 1.5, 5.0, 64)}, 160, 0.11),
            layer(4, 4, 64, 130, {"base": 1.0e4, "dims": 64}, 192, 0.15),
            layer(2, 1, 128, 96, {"base": 3.0e4, "dims": 16}, 0, 0.07)]}
# PLAIN: neither chunks nor rotation nor cap in one layer: the switches' other position.
BARE = {"architecture": "Mekazen", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "logit_softcap": None,
        "layers": [layer(2, 2, 32, 0, None, 64, 0.25), layer(4, 2, 16, 9, {"base": 50.0, "dims": 16}, 40, 0.5)]}
MODELS = {"small": (SMALL, 11, 8, 1.0), "wide": (WIDE, 12, 16, 1.0), "bare": (BARE, 13, 4, 1.0),
          # the query and key norms' factors twice as large: scores four times as far apart, so that which
          # keys a query sees decides its output. Rounding grows with the scores too: float32 only, a bound
          # of its own.
          "sharp": (SMALL, 14, 8, 2.0)}   # name -> configuration, seed, page size, factor on the q/k norms
CASES = [(name, dtype) for name in MODELS for dtype in ("float32", "bfloat16") if (name, dtype) != ("sharp", "bfloat16")]

TOL = {"float32": 4e-5, "bfloat16": 1e-1}        # engine against plain (float64), logits of a few units
TOL_CUTS = {"float32": 2e-5, "bfloat16": 1e-1}   # the engine against itself, however the work is cut
TOL_SHARP = 5e-4


def bound(name, dtype, cuts_only=False):
    if name == "sharp":
        return TOL_SHARP
    return (TOL_CUTS if cuts_only else TOL)[dtype]


def write_folder(folder, raw, seed, sharpen):
    """config.json + model.safetensors: bfloat16 matrices, float32 norm weights
    (so that the engine and the plain side hold the same values), the output
    head eight times larger (logits of a few units, which the cap bends)."""
    from metallix_b200.config import MekazenConfig
    from metallix_b200.weights import random_tensors
    from metallix_b200.weights.safetensors_io import write_file
    config = MekazenConfig.from_dict(raw)
    tensors = random_tensors(config, seed, dtype="bfloat16", norm_dtype="float32")
    tensors["head"] = (tensors["head"].float() * 8.0).to(torch.bfloat16)
    for name in tensors:
        if name.endswith(".q.norm") or name.endswith(".k.norm"):
            tensors[name] = tensors[name] * sharpen
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config.to_dict(), handle)
    write_file(os.path.join(folder, "model.safetensors"), {k: v.cpu() for k, v in tensors.items()},
               order=list(config.tensor_shapes()))
    return folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """name -> (folder, config dict, tensors as float64 numpy, page size)."""
    out = {}
    for name, (raw, seed, page, sharpen) in MODELS.items():
        folder = write_folder(str(tmp_path_factory.mktemp(f"mekazen_{name}")), raw, seed, sharpen)
        config, tensors = plain.read_model(folder)
        out[name] = (folder, config, tensors, page)
    return out


def make_engine(folders, name, dtype, pages=96, **options):
    from metallix_b200.engine import Engine
    folder, _, _, page = folders[name]
    return Engine.from_folder(folder, dtype=dtype, page_tokens=page, num_pages=pages,
                              max_requests=options.pop("max_requests", 8), **options)


# ------------------------------------------------ configuration (no GPU needed)
def test_configuration_round_trip_and_registry():
    from metallix_b200.config import ConfigError, MekazenConfig, parse_config, resolve
    for raw in (SMALL, WIDE, BARE):
        config = parse_config(raw)
        assert isinstance(config, MekazenConfig) and resolve(raw).kind == "mekazen"
        assert MekazenConfig.from_dict(config.to_dict()) == config
        assert json.loads(json.dumps(config.to_dict())) == config.to_dict()
        shapes = config.tensor_shapes()
        for index, spec in enumerate(raw["layers"]):
            mixer = spec["mixer"]
            assert shapes[f"l{index}.mix.q"] == (mixer["heads"] * mixer["dim"], raw["width"])
            assert shapes[f"l{index}.mix.k"] == (mixer["kv_heads"] * mixer["dim"], raw["width"])
            assert shapes[f"l{index}.mix.k.norm"] == (mixer["kv_heads"] * mixer["dim"],)
            assert (f"l{index}.mlp.up" in shapes) == bool(spec["mlp"])
            assert (f"l{index}.norm2b" in shapes) == bool(spec["mlp"])
            assert f"l{index}.mix.v" not in shapes
        model = config.to_model_spec()
        assert [bool(l.feed_forward) for l in model.layers] == [bool(s["mlp"]) for s in raw["layers"]]
        assert [l.mixer.get("chunk") for l in model.layers] == \
            [(s["mixer"].get("mask") or {}).get("size") for s in raw["layers"]]
    refusals = [
        ("UnsupportedLayerType", lambda c: c["layers"][0].update(type="recurrent")),
        ("InvalidValueWidth", lambda c: c["layers"][0]["mixer"].update(vdim=8)),
        ("InvalidGroupedQueryLayout", lambda c: c["layers"][0]["mixer"].update(kv_heads=3)),
        ("InvalidRotaryWidth", lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18)),
        ("UnsupportedFeedForward", lambda c: c["layers"][0]["mlp"].update(kind="routed")),
        ("MissingDimension", lambda c: c.update(width=0)),
        ("MissingDimension", lambda c: c.update(layers=[])),
        ("UnsupportedRopeScaling", lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(high=0.25))]
    for kind, change in refusals:
        raw = json.loads(json.dumps(SMALL))
        change(raw)
        with pytest.raises(ConfigError) as caught:
            parse_config(raw)
        assert caught.value.kind == kind


def test_random_weights_follow_how_a_norm_is_stored(tmp_path):
    """Zero-centred norms are drawn about zero, the query and key norms
    about one; a checkpoint with a tensor too many or of the wrong shape is refused."""
    from metallix_b200.config import MekazenConfig
    from metallix_b200.weights import CheckpointError, load_tensors, random_tensors, write_model_folder
    config = MekazenConfig.from_dict(SMALL)
    tensors = random_tensors(config, 3, dtype="float32")
    assert abs(float(tensors["l0.norm1"].mean())) < 0.05 and float(tensors["l0.norm1"].abs().max()) <= 0.1
    assert abs(float(tensors["final.norm"].mean())) < 0.05
    assert abs(float(tensors["l2.mix.q.norm"].mean()) - 1.0) < 0.05
    folder = write_model_folder(str(tmp_path / "m"), config, 3)
    loaded = load_tensors(folder, config)
    assert set(loaded) == set(config.tensor_shapes()) and "l1.norm2" not in loaded
    other = json.loads(json.dumps(SMALL))
    other["layers"][1]["mixer"]["kv_heads"] = 1
    with pytest.raises(CheckpointError):
        load_tensors(folder, MekazenConfig.from_dict(other))


def test_frequencies_in_three_bands():
    """The engine's frequencies against the plain side's, with pairs in each of
    the three bands (kept, divided, blended) and without a stretch."""
    from metallix_b200.parts.position import rotary_frequencies
    for base, dims, scaling in ((1.0e4, 32, bands(4.0, 0.5, 3.0, 40)), (1.0e6, 64, bands(8.0, 1.5, 5.0, 1000)),
                                (1.0e2, 2, bands(2.5, 2.0, 16.0, 100)), (5.0e3, 24, None)):
        want = plain.pair_frequencies(base, dims, scaling)
        got = rotary_frequencies(base, dims, scaling).numpy()
        assert np.allclose(got, want, rtol=1e-14, atol=0.0)
        if scaling and dims > 2:
            bare = plain.pair_frequencies(base, dims, None)
            ratio = want / bare
            kept, divided = np.isclose(ratio, 1.0), np.isclose(ratio, 1.0 / scaling["factor"])
            assert kept.any() and divided.any() and (~kept & ~divided).any()


def test_chunked_groups_give_pages_back():
    """The cache manager returns the pages of chunks that no later query sees,
    hands them out again, and keeps its books through all of it."""
    from metallix_b200.csrc import build
    host = build.host()
    manager = host.CacheManager([host.GroupConfig(4, 0, 24, 10), host.GroupConfig(4, 0, 24, 0),
                                 host.GroupConfig(4, 6, 24, 10)], 2)
    manager.admit(1)
    held = []
    for step in range(40):
        manager.reserve(1, 1)
        manager.commit(1, 1)
        manager.check_invariants()
        computed = step + 1
        held.append([sum(1 for page in manager.table(1, g) if page >= 0) for g in range(3)])
        # chunks of 10: pages wholly before the chunk of the next position are gone
        first_needed = computed - computed % 10
        assert manager.first_live_page(1, 0) == first_needed // 4
        assert manager.first_live_page(1, 1) == 0
        # window 6 and chunks of 10 together: the later of the two first keys
        assert manager.first_live_page(1, 2) == max(first_needed, computed - 6 + 1, 0) // 4
    assert max(h[0] for h in held) <= 4 and held[-1][1] == 10
    assert manager.pages_reused() > 0
    manager.admit(2)
    manager.reserve(2, 33)          # a prompt that crosses three chunk edges in one step
    manager.commit(2, 33)
    assert manager.first_live_page(2, 0) == 30 // 4
    manager.release(1)
    manager.release(2)
    manager.check_invariants()
    assert [manager.free_pages(g) for g in range(3)] == [24, 24, 24]


def test_the_plain_side_one_position_at_a_time():
    """The plain implementation itself: a sequence's logits do not change when
    more tokens follow, and a chunk's first position sees only itself."""
    folder_config = json.loads(json.dumps(BARE))
    rng = np.random.default_rng(0)
    from metallix_b200.config import MekazenConfig
    shapes = MekazenConfig.from_dict(folder_config).tensor_shapes()
    tensors = {name: rng.normal(size=shape) * (0.1 if len(shape) == 1 else 0.3) for name, shape in shapes.items()}
    ids = random_ids(1, 30, 97)
    whole = plain.forward_logits(folder_config, tensors, ids)
    assert np.allclose(plain.forward_logits(folder_config, tensors, ids[:19]), whole[:19], atol=1e-12)
    q = rng.normal(size=(20, 2, 4))
    k = rng.normal(size=(20, 1, 4))
    v = rng.normal(size=(20, 1, 4))
    out = plain.masked_attention(q, k, v, list(range(20)), 0.5, 9)
    assert np.allclose(out[9], v[9, 0]) and np.allclose(out[18], v[18, 0]) and not np.allclose(out[17], v[17, 0])


# --------------------------------------------------------- mechanisms alone
gpu = pytest.mark.gpu


def dev(array, dtype=torch.float32):
    return torch.tensor(np.asarray(array), dtype=dtype, device="cuda")


def rounded(array, dtype):
    return torch.tensor(np.asarray(array), dtype=dtype).double().numpy()


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, dim, dims, interleaved", [
    (4, 2, 16, 8, True), (3, 3, 24, 24, True), (6, 1, 12, 2, True), (2, 1, 128, 16, True), (8, 2, 64, 64, True),
    (5, 5, 20, 10, False)])
def test_norm_over_the_projection_rotation_and_cache(dtype, heads, kv_heads, dim, dims, interleaved):
    """One kernel: RMS norm over all of a token's query values (and all of its
    key values), rotation of pairs over the first ``dims`` values of each head,
    q out, rotated keys and the untouched values into the cache at the slots."""
    from metallix_b200 import ops
    from metallix_b200.parts.position import rotary_frequencies
    rng = np.random.default_rng(heads * dim + dims)
    tokens, page, pages, eps = 37, 8, 9, 1e-5
    scaling = bands(4.0, 0.5, 3.0, 40)
    positions = rng.permutation(60)[:tokens]
    wide = rounded(rng.normal(size=(tokens, (heads + kv_heads) * dim + 8)), dtype)   # q and k as column ranges
    q, k = wide[:, :heads * dim], wide[:, heads * dim:(heads + kv_heads) * dim]
    q_gain, k_gain = rng.uniform(0.5, 1.5, heads * dim), rng.uniform(0.5, 1.5, kv_heads * dim)
    frequency = rotary_frequencies(1.0e4, dims, scaling)
    angle = torch.arange(64, dtype=torch.float64)[:, None] * frequency[None, :]
    cos, sin = torch.cos(angle).float().cuda().contiguous(), torch.sin(angle).float().cuda().contiguous()
    slots = rng.permutation(page * pages)[:tokens]
    slots[5] = -1   # a token that writes nothing
    device_wide = dev(wide, dtype)
    q_dev, k_dev = device_wide[:, :heads * dim], device_wide[:, heads * dim:(heads + kv_heads) * dim]
    q_out = torch.empty((tokens, heads, dim), dtype=dtype, device="cuda")
    cache = torch.full((pages, 2, kv_heads, page, dim), 7.0, dtype=dtype, device="cuda")
    ops.qk_norm_rope_cache(q_dev, k_dev, k_dev, q_out, cache, dev(slots, torch.int32), dev(positions, torch.int32),
                           dev(q_gain), dev(k_gain), cos, sin, eps, interleaved=interleaved, norm_scope="projection")
    ops.check_status("cuda")
    gain_q, gain_k = dev(q_gain).double().cpu().numpy(), dev(k_gain).double().cpu().numpy()
    want_q = plain.norm_plain(q, gain_q, eps).reshape(tokens, heads, dim)
    want_k = plain.norm_plain(k, gain_k, eps).reshape(tokens, kv_heads, dim)
    if interleaved:
        want_q = plain.rotate_pairs(want_q, positions, 1.0e4, dims, scaling)
        want_k = plain.rotate_pairs(want_k, positions, 1.0e4, dims, scaling)
    else:   # halves: value i with value i + dims / 2
        def halves(x):
            out, half = x.copy(), dims // 2
            f = plain.pair_frequencies(1.0e4, dims, scaling)
            for t, p in enumerate(positions):
                c, s = np.cos(p * f), np.sin(p * f)
                out[t, :, :half] = x[t, :, :half] * c - x[t, :, half:dims] * s
                out[t, :, half:dims] = x[t, :, half:dims] * c + x[t, :, :half] * s
            return out
        want_q, want_k = halves(want_q), halves(want_k)
    bound = 1e-5 if dtype == torch.float32 else 3e-2
    assert np.abs(q_out.double().cpu().numpy() - want_q).max() < bound
    got = cache.double().cpu().numpy()
    untouched = np.ones((pages, page), dtype=bool)
    for t, slot in enumerate(slots):
        if slot < 0:
            continue
        untouched[slot // page, slot % page] = False
        assert np.abs(got[slot // page, 0, :, slot % page] - want_k[t]).max() < bound
        assert np.array_equal(got[slot // page, 1, :, slot % page], k[t].reshape(kv_heads, dim))   # as projected
    assert (got.transpose(0, 3, 1, 2, 4)[untouched] == 7.0).all()


@gpu
@pytest.mark.parametrize("size, rows, parts", [(72, 5, 1), (128, 3, 6), (331, 2, 1), (4096, 4, 3)])
@pytest.mark.parametrize("delta_dtype", [torch.float32, torch.bfloat16])
def test_norm_behind_a_sublayer_sum_and_next_norm(size, rows, parts, delta_dtype):
    """x += norm(d) * (1 + w1); y = norm(x) * (1 + w2) in one kernel, d whole or
    in parts, with and without the second norm."""
    from metallix_b200 import ops
    if parts > 1 and delta_dtype != torch.float32:
        pytest.skip("parts are float32")
    rng = np.random.default_rng(size + parts)
    x = rng.normal(size=(rows, size)) * 3.0
    delta = rounded(rng.normal(size=(parts, rows, size)) * 20.0, delta_dtype)
    w1, w2 = rng.uniform(-0.3, 0.3, size), rng.uniform(-0.3, 0.3, size)
    f32 = lambda a: dev(a).double().cpu().numpy()
    summed = np.zeros((rows, size), dtype=np.float32)
    for part in delta:
        summed = summed + part.astype(np.float32)     # the kernel adds the parts up in float32, in their order
    want_x = f32(x) + plain.norm_around_zero(summed.astype(np.float64), f32(w1), 1e-6)
    want_y = plain.norm_around_zero(want_x, f32(w2), 1e-5)
    for out_dtype in (torch.float32, torch.bfloat16):
        x_dev = dev(x)
        d_dev = dev(delta if parts > 1 else delta[0], delta_dtype)
        y = ops.postnorm_add_rmsnorm(x_dev, d_dev, dev(1.0 + f32(w1)), 1e-6, dev(1.0 + f32(w2)), 1e-5, out_dtype)
        assert np.abs(x_dev.double().cpu().numpy() - want_x).max() < 2e-5
        assert np.abs(y.double().cpu().numpy() - want_y).max() < (1e-5 if out_dtype == torch.float32 else 3e-2)
    x_dev = dev(x)
    assert ops.postnorm_add_rmsnorm(x_dev, dev(delta if parts > 1 else delta[0], delta_dtype),
                                    dev(1.0 + f32(w1)), 1e-6) is None
    assert np.abs(x_dev.double().cpu().numpy() - want_x).max() < 2e-5


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_output_gate_and_capped_logits(dtype):
    from metallix_b200 import ops
    rng = np.random.default_rng(5)
    wide = rounded(rng.normal(size=(9, 200)) * 3.0, dtype)
    a = rounded(rng.normal(size=(9, 72)), dtype)
    wide_dev = dev(wide, dtype)
    out = ops.sigmoid_gate(dev(a, dtype), wide_dev[:, 100:172])
    want = a / (1.0 + np.exp(-wide[:, 100:172]))
    assert np.abs(out.double().cpu().numpy() - want).max() < (1e-6 if dtype == torch.float32 else 1e-2)
    logits = rng.normal(size=(4, 333)) * 20.0
    got = ops.softcap_(dev(logits), 7.5).double().cpu().numpy()
    assert np.abs(got - plain.capped(dev(logits).double().cpu().numpy(), 7.5)).max() < 2e-6
    assert np.abs(got).max() < 7.5 + 1e-6


# ------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def references(folders):
    """name -> (requests: id -> token ids, plain logits per request, residual stream per layer of 'r0')."""
    out = {}
    for name, (folder, config, tensors, page) in folders.items():
        lengths = (150, 61, 1, 9, 100, 33) if name != "wide" else (300, 140, 1, 9, 70, 33)
        requests = {f"r{i}": random_ids(100 + 7 * i, n, config["vocab"]) for i, n in enumerate(lengths)}
        layers = []
        logits = {}
        for key, ids in requests.items():
            logits[key] = plain.forward_logits(config, tensors, ids, keep=layers if key == "r0" else None)
        out[name] = (requests, logits, layers)
    return out


@gpu
@pytest.mark.parametrize("name, dtype", CASES)
def test_whole_prompts_and_every_layer(folders, references, name, dtype):
    """Each request in one step; for one of them the residual stream after
    every layer (float32: each layer is right, not only their sum)."""
    from metallix_b200.engine import StepEntry
    requests, logits, layers = references[name]
    engine = make_engine(folders, name, dtype)
    worst, _ = cuts.replay(engine, cuts.whole(requests), logits, StepEntry)
    assert worst < bound(name, dtype), worst
    seen = []
    engine.step([StepEntry("tap", requests["r0"], [])], tap=lambda index, residual: seen.append(residual.clone()))
    engine.check()
    assert len(seen) == len(layers)
    for index, (got, want) in enumerate(zip(seen, layers)):
        scale = np.abs(want).max()
        limit = (2e-5 if dtype == "float32" else 4e-2) * (10 if name == "sharp" else 1)
        assert np.abs(got.double().cpu().numpy() - want).max() < limit * scale, index
    engine.release_all()
    engine.manager.check_invariants()


@gpu
@pytest.mark.parametrize("name, dtype", CASES)
def test_decoding_portions_and_mixed_batches(folders, references, name, dtype):
    """The same requests: most of a prompt and then its last tokens one by one
    (over several chunk edges), portions of changing size down to two tokens,
    and up to four live requests in one step with a pool made for the most
    tokens live at a time, so that pages are used again. Every way agrees with
    the plain side and, within rounding, with the whole prompts."""
    from metallix_b200.engine import StepEntry
    requests, logits, _ = references[name]
    page = folders[name][3]
    engine = make_engine(folders, name, dtype)
    _, whole = cuts.replay(engine, cuts.whole(requests), logits, StepEntry)
    ways = {"tail": cuts.tail_by_one(requests, tail=60), "ragged": cuts.ragged(requests)}
    mixed, peak = cuts.mixed(requests, 3)
    for way, steps in ways.items():
        worst, seen = cuts.replay(engine, steps, logits, StepEntry)
        assert worst < bound(name, dtype), (way, worst)
        gap = max(float(np.abs(row - whole[key]).max()) for key, row in seen.items())
        assert gap < bound(name, dtype, cuts_only=True), (way, gap)
    engine.release_all()
    small = make_engine(folders, name, dtype, pages=peak // page + 4 * (64 // page), max_requests=4)
    worst, seen = cuts.replay(small, mixed, logits, StepEntry)
    assert worst < bound(name, dtype), worst
    gap = max(float(np.abs(row - whole[key]).max()) for key, row in seen.items())
    assert gap < bound(name, dtype, cuts_only=True), gap
    assert small.manager.pages_reused() > 0
    small.manager.check_invariants()
    assert small.manager.live_requests() == 0


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_pool_smaller_than_the_sequence(folders, dtype):
    """Every layer of the small model has chunks of at most 40 positions, so a
    request never needs more than a chunk's pages and the one being filled:
    220 positions pass through a pool of 10 pages of 8, as a prompt in portions
    and then token by token, through decode graphs, beside a second request."""
    from metallix_b200.engine import StepEntry
    _, config, tensors, page = folders["small"]
    ids = {"a": random_ids(41, 220, config["vocab"]), "b": random_ids(42, 90, config["vocab"])}
    want = {key: plain.forward_logits(config, tensors, value) for key, value in ids.items()}
    engine = make_engine(folders, "small", dtype, pages=14, max_requests=2)
    worst, at = 0.0, {"a": 0, "b": 0}

    def step(entries):
        nonlocal worst
        logits = engine.step([StepEntry(key, ids[key][at[key]:at[key] + n], [n - 1]) for key, n in entries])
        got = logits.double().cpu().numpy()
        for row, (key, n) in enumerate(entries):
            at[key] += n
            worst = max(worst, float(np.abs(got[row] - want[key][at[key] - 1]).max()))

    for size in (30, 17, 2, 21):
        step([("a", size)])
    step([("a", 1), ("b", 33)])
    while at["a"] < 220:
        live = [("a", 1)] + ([("b", 1)] if at["b"] < 90 else [])
        step(live)
        if at["b"] == 90 and engine.live("b"):
            engine.release("b")
    engine.check()
    assert worst < TOL[dtype], worst
    assert engine.manager.pages_reused() > 20
    engine.manager.check_invariants()
    engine.release_all()
    assert [engine.manager.free_pages(g) for g in range(engine.manager.num_groups())] == \
        [14] * engine.manager.num_groups()


@gpu
@pytest.mark.parametrize("name", ["small", "wide"])
def test_a_batch_gives_what_each_request_gives_alone(folders, references, name):
    """float32: unequal requests in one step (a prompt, a portion behind cached
    tokens, single tokens) against each of them alone, bit for bit where one
    kernel family serves both (the general kernels of the small model)."""
    from metallix_b200.engine import StepEntry
    requests, logits, _ = references[name]
    keys = ["r0", "r1", "r3", "r4"]
    alone = make_engine(folders, name, "float32", cuda_graphs=False)
    single = {}
    for key in keys:
        ids = requests[key]
        cutoff = len(ids) // 2
        alone.step([StepEntry(key, ids[:cutoff], [])])
        single[key] = alone.step([StepEntry(key, ids[cutoff:], list(range(len(ids) - cutoff)))]).clone()
        alone.release(key)
    batch = make_engine(folders, name, "float32", cuda_graphs=False)
    batch.step([StepEntry(key, requests[key][:len(requests[key]) // 2], []) for key in keys])
    together = batch.step([StepEntry(key, requests[key][len(requests[key]) // 2:],
                                     list(range(len(requests[key]) - len(requests[key]) // 2))) for key in keys])
    row = 0
    for key in keys:
        count = single[key].shape[0]
        got, want = together[row:row + count], single[key]
        if name == "small":
            assert torch.equal(got, want), key
        else:
            assert float((got - want).abs().max()) < TOL_CUTS["float32"], key
        row += count
    batch.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_of_a_sequence(folders, dtype):
    """A prompt of one token, then decoding from position 1; a request that
    joins a running batch with its first token; slots that are used again."""
    from metallix_b200.engine import StepEntry
    _, config, tensors, _ = folders["bare"]
    engine = make_engine(folders, "bare", dtype, pages=64, max_requests=2)
    for turn in range(3):      # the same two slots, three times over
        ids = {"x": random_ids(60 + turn, 12, config["vocab"]), "y": random_ids(70 + turn, 6, config["vocab"])}
        want = {key: plain.forward_logits(config, tensors, value) for key, value in ids.items()}
        for position in range(12):
            entries = [StepEntry("x", [ids["x"][position]], [0])]
            if 3 <= position < 9:
                entries.append(StepEntry("y", [ids["y"][position - 3]], [0]))
            got = engine.step(entries).double().cpu().numpy()
            assert np.abs(got[0] - want["x"][position]).max() < TOL[dtype], (turn, position)
            if len(entries) > 1:
                assert np.abs(got[1] - want["y"][position - 3]).max() < TOL[dtype], (turn, position)
            if position == 8:
                engine.release("y")
        engine.release("x")
    engine.check()


@gpu
def test_sharp_scores_show_a_chunk_edge_that_is_one_off(folders, references):
    """What the sharp model is for: had the engine put a chunk's edge one
    position off, or left the chunks out, its logits would be far outside the
    bound that the other tests hold it to."""
    _, config, tensors, _ = folders["sharp"]
    requests, logits, _ = references["sharp"]
    ids = requests["r0"]
    for change in (1, -1, None):
        other = json.loads(json.dumps(config))
        for spec in other["layers"]:
            if change is None:
                spec["mixer"]["mask"] = None
            else:
                spec["mixer"]["mask"]["size"] += change
        wrong = plain.forward_logits(other, tensors, ids)
        assert np.abs(wrong - logits["r0"]).max() > 100 * TOL_SHARP, change


# ------------------------------------------------- scheduler, command line
@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(folders, dtype):
    """``generate``: continuous batching, prompts in portions, decode graphs;
    the tokens are the plain side's greedy tokens (bfloat16: up to a near tie)."""
    from metallix_b200.engine.generate import generate
    _, config, tensors, _ = folders["wide"]
    prompts = [random_ids(80 + i, n, config["vocab"]) for i, n in enumerate((5, 61, 1, 40))]
    engine = make_engine(folders, "wide", dtype, pages=64)
    results = generate(engine, prompts, max_new_tokens=14, eos_ids=(), max_num_seqs=3, prefill_chunk=24,
                       max_tokens_per_step=48)
    for prompt, result in zip(prompts, results):
        assert result.finish_reason == "length" and len(result.generated_ids) == 14
        ids = list(prompt)
        for step, token in enumerate(result.generated_ids):
            row = plain.forward_logits(config, tensors, ids)[-1]
            best = int(np.argmax(row))
            if token != best:
                assert dtype == "bfloat16" and row[best] - row[token] < 0.1, (step, token, best)
                break
            ids.append(token)
    assert engine.manager.live_requests() == 0
    engine.manager.check_invariants()


@gpu
def test_command_line_and_trace_program(folders, references, tmp_path):
    """``mxb gen --model`` on a Mekazen folder (greedy, cache verified against
    the second kernel family) and ``trace_run`` on a mixed schedule."""
    folder, config, tensors, page = folders["wide"]
    prompt = random_ids(90, 23, config["vocab"])
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "mxb"), "gen", "--model", folder, "--input-ids",
                          ",".join(map(str, prompt)), "--max-tokens", "6", "--dtype", "float32", "--verify-cache"],
                         capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    receipt = json.loads(run.stdout.strip().splitlines()[-1])
    assert receipt["generated_ids"] == plain.greedy(config, tensors, prompt, 6)
    assert receipt["operation"] == "mekazen_greedy_cached_generation"
    assert receipt["cache_comparisons"]["logits_within_bound"]
    requests, logits, _ = references["wide"]
    steps, peak = cuts.mixed(requests, 9)
    out = tmp_path / "trace"
    text = "".join(json.dumps(step) + "\n" for step in steps)
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype",
                          "bfloat16", "--out", str(out), "--max-tokens", str(peak)],
                         input=text, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [line for line in run.stdout.splitlines() if line.startswith("done")] == \
        [f"done {step['step']}" for step in steps]
    offsets = {}
    for step in steps:
        for entry in step["entries"]:
            offsets.setdefault(entry["id"], 0)
        want = cuts.expected_rows(step, offsets, logits)
        if want is not None:
            got = np.fromfile(out / f"{step['step']}.f32", dtype="<f4").reshape(-1, config["vocab"])
            assert np.abs(got - want).max() < TOL["bfloat16"], step["step"]
        for entry in step["entries"]:
            offsets[entry["id"]] += len(entry["tokens"])
