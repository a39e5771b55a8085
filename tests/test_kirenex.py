"""Kirenex without a device: configuration, the spec's tensors and parts, the rotation's frequencies, and what
the cache manager makes of kept first tokens, of a latent that two layers read and of a mixer made of two."""

import json

import pytest
import torch

import layover_b200 as lb
import plain_kirenex as plain
from kirenex_configs import CONFIGS, config, latent, left, parallel, right
from layover_b200.cache import CacheManager
from layover_b200.config.base import load_config, resolve_architecture
from layover_b200.models import assemble, spec_for_config
from layover_b200.parts.base import PagedKVNeed, PartSpec, Runtime, StateNeed, build_part


@pytest.mark.parametrize("name", list(CONFIGS))
def test_config_round_trip_and_registry(name, tmp_path):
    raw = CONFIGS[name]
    cfg = lb.KirenexConfig.from_hf_dict(raw)
    assert lb.KirenexConfig.from_hf_dict(cfg.to_hf_dict()) == cfg
    assert resolve_architecture(raw).config_class is lb.KirenexConfig
    (tmp_path / "config.json").write_text(json.dumps(raw))
    arch, again = load_config(tmp_path)
    assert arch.name == "Kirenex" and again == cfg


def test_refusals():
    good = CONFIGS["odd_sizes"]
    for change, match in [
        (lambda c: c["layers"][0].update(type="attention"), "unknown type"),
        (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
        (lambda c: c["layers"][0]["mixer"].update(rot_dim=5), "rot"),
        (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=4), "rot.dims must equal rot_dim"),
        (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier layer"),
        (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "latent_attention layer"),
        (lambda c: c["layers"][2]["mixer"].update(kv_rank=40), "must equal those of layer 0"),
        (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "multiple of kv_heads"),
        (lambda c: c["layers"][1]["mixer"]["right"].update(heads=3), "multiple of kv_heads"),
        (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=14), "rot"),
        (lambda c: c["layers"][1]["mixer"]["left"]["rot"]["scaling"].pop("high"), "scaling lacks"),
        (lambda c: c["layers"][1]["mixer"]["left"]["mask"].update(size=0), "mask.size"),
        (lambda c: c["layers"][1]["mixer"]["left"]["mask"].update(keep_first=-1), "keep_first"),
        (lambda c: c["layers"][1]["mixer"]["right"].update(conv=0), "conv"),
        (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "mlp kind"),
        (lambda c: c.update(postln_alpha=0.0), "postln_alpha"),
        (lambda c: c.pop("max_positions"), "lacks"),
    ]:
        raw = json.loads(json.dumps(good))
        change(raw)
        with pytest.raises(ValueError, match=match):
            lb.KirenexConfig.from_hf_dict(raw)


def test_the_specs_tensors_have_the_checkpoints_names_and_shapes():
    raw = config(50, 24, [
        latent(3, 4, 2, 6, 10, 100.0, 0.3, ff=14),
        parallel(left(4, 2, 8, 6, 5, 2, 4, 100.0, 0.1), right(4, 2, 6, 10, 3), ff=18),
        latent(2, 8, 2, 4, 10, 100.0, 0.2, kv_from=0),
    ], alpha=2.5, positions=77)
    spec = spec_for_config(lb.KirenexConfig.from_hf_dict(raw))
    specs = {s.name: tuple(s.shape) for s in spec.tensor_specs()}
    want = {"embed": (50, 24), "pos": (77, 24), "head": (50, 24), "final.norm": (24,),
            "l0.norm1": (24,), "l0.norm2": (24,), "l1.norm1": (24,), "l1.norm2": (24,), "l2.norm1": (24,),
            "l0.mix.q": (3 * 6, 24), "l0.mix.dkv": (12, 24), "l0.mix.dkv.norm": (10,), "l0.mix.uk": (3 * 4, 10),
            "l0.mix.uv": (3 * 6, 10), "l0.mix.g": (3 * 6, 24), "l0.mix.o": (24, 3 * 6),
            "l2.mix.q": (2 * 10, 24), "l2.mix.uk": (2 * 8, 10), "l2.mix.uv": (2 * 4, 10), "l2.mix.g": (2 * 4, 24),
            "l2.mix.o": (24, 2 * 4),
            "l1.mix.left.q": (32, 24), "l1.mix.left.k": (16, 24), "l1.mix.left.v": (12, 24), "l1.mix.left.q.norm": (8,),
            "l1.mix.left.k.norm": (8,), "l1.mix.left.o": (24, 24), "l1.mix.left.out": (24,), "l1.mix.right.out": (24,),
            "l1.mix.right.q": (12, 24), "l1.mix.right.k": (12, 24), "l1.mix.right.v": (40, 24),
            "l1.mix.right.q.conv": (12, 3), "l1.mix.right.k.conv": (12, 3), "l1.mix.right.v.conv": (40, 3),
            "l1.mix.right.b": (4, 24), "l1.mix.right.a": (4, 24), "l1.mix.right.A_log": (4,), "l1.mix.right.dt_bias": (4,),
            "l1.mix.right.g": (40, 24), "l1.mix.right.norm": (10,), "l1.mix.right.o": (24, 40),
            "l0.mlp.gate": (14, 24), "l0.mlp.up": (14, 24), "l0.mlp.down": (24, 14),
            "l1.mlp.gate": (18, 24), "l1.mlp.up": (18, 24), "l1.mlp.down": (24, 18)}
    assert specs == want
    assert spec.residual_dtype == "float32" and spec.max_position == 77 and spec.position_table == "pos"
    assert [entry.reads_cache_of for entry in spec.schedule] == [None, None, 0]
    model = assemble(spec)
    assert [type(block).__name__ for block in model.blocks] == ["PostNormBlock"] * 3
    assert [block.alpha for block in model.blocks] == [2.5] * 3
    assert model.blocks[2].feed_forward is None and model.blocks[2].ff_norm is None
    window = model.blocks[1].mixer.mixers[0]
    assert (window.window, window.keep_first, window.position.rotated, window.scale) == (5, 2, 4, 0.1)


@pytest.mark.parametrize("base, dims, scaling", [
    (300.0, 8, (4.0, 1.0, 4.0, 64)), (20000.0, 16, (8.0, 1.0, 2.0, 32)), (10000.0, 16, (2.0, 1.0, 8.0, 16)),
    (10000.0, 32, None), (50.0, 12, (3.0, 0.5, 6.0, 40))])
def test_banded_frequencies(base, dims, scaling):
    table = dict(zip(("factor", "low", "high", "original"), scaling)) if scaling else None
    want = plain.banded_frequencies(base, dims, table)
    if scaling:       # the cases are made so that the bands they name are in use
        plain_f = plain.plain_frequencies(base, dims)
        assert bool((want != plain_f).any())
    for kind in ("rotary_half", "rotary_pairs"):
        part = build_part("position", PartSpec(kind, {"dim": dims + 8, "theta": base, "rotated": dims, "band_scaling": table}), "")
        part.bind({}, Runtime(torch.float32, torch.device("cpu"), None))
        assert torch.allclose(part.inv_freq().double(), want, rtol=1e-6, atol=0)


def test_the_cache_of_a_model_with_every_kind_of_layer():
    raw = CONFIGS["wide_heads"]
    model = assemble(spec_for_config(lb.KirenexConfig.from_hf_dict(raw)))
    needs = model.cache_needs()
    # before the parts are bound they ask for the 32-bit path's rooms (multiples of 4)
    assert needs[1][1] == PagedKVNeed(1, 64, values_in_keys=True) and needs[1][2] is None
    assert [reads for _, _, reads in needs] == [None, None, 1, None, 1]
    first = needs[0][1]
    assert isinstance(first, tuple) and first[0] == PagedKVNeed(1, 32, 7, 16, keep_first=16)
    assert first[1] == StateNeed((2 * 32 * 48 + 2 * (2 * 32 + 2 * 48),), torch.float32)
    cache = CacheManager(needs, 12, 16, torch.float32, "cpu", max_requests=2)
    assert [g.entries for g in cache.paged] == [[0], [1], [3]] and [g.entries for g in cache.states] == [[0], [3]]
    assert cache.view(0).kind == "composite" and [v.kind for v in cache.view(0).parts] == ["paged", "state"]
    # the layers that read layer 1's latent see its pool, and write nothing
    for reader in (2, 4):
        places = {cache.view(reader).k_pool.data_ptr(), cache.view(reader).v_pool.data_ptr(), cache.view(1).k_pool.data_ptr(),
                  cache.view(1).v_pool.data_ptr()}
        assert len(places) == 1 and not cache.view(reader).writes and cache.view(1).writes
    assert cache.paged[1].k_store.shape == (1, 13, 1, 16, 64) and cache.paged[1].v_store is None


@pytest.mark.parametrize("window, keep, page", [(7, 16, 16), (24, 5, 4), (9, 0, 4), (1, 2, 2), (40, 3, 16), (6, 9, 4)])
def test_kept_first_tokens_keep_their_pages(window, keep, page):
    need = PagedKVNeed(1, 8, window, keep_first=keep)
    cache = CacheManager([(0, need, None)], 64, page, torch.float32, "cpu", max_requests=2)
    group = cache.paged[0]

    def visible_pages(total):       # pages that hold a key some query at position >= total can see
        live = set(range(max(0, total - window + 1) // page, -(-total // page)))
        return live | set(range(-(-min(keep, total) // page)))

    seq = cache.open("a")
    for total in range(1, 150):
        cache.grow(seq, total)
        cache.commit(seq, total)
        cache.check()
        table = seq.tables[0]
        held = {i for i, b in enumerate(table.blocks) if b != group.scratch_page}
        assert held == visible_pages(total), total
        assert table.given_back == len(table.blocks) - len(held)
    most = max(1, window - 1 + 1) // page + 2 + -(-keep // page)
    assert cache.peak_blocks(0, 149, 1) == min(cache.blocks_for(149), most)
    # a long portion: everything it can see stays until the step is done, then all of it goes at once
    other = cache.open("b")
    cache.grow(other, 3); cache.commit(other, 3)
    cache.grow(other, 100)
    assert {i for i, b in enumerate(other.tables[0].blocks) if b != group.scratch_page} == set(range(-(-100 // page)))
    cache.commit(other, 100)
    assert {i for i, b in enumerate(other.tables[0].blocks) if b != group.scratch_page} == visible_pages(100)
    cache.close(seq); cache.close(other); cache.check()
    assert group.allocator.num_used == 0
    # the pages that went back are handed out again, and the new owner's kept pages stay its own
    again = cache.open("c")
    cache.grow(again, 70); cache.commit(again, 70); cache.check()
    assert {i for i, b in enumerate(again.tables[0].blocks) if b != group.scratch_page} == visible_pages(70)
    cache.close(again)


def test_presets_and_random_folders(tmp_path):
    cfg = lb.preset("kirenex-tiny")
    assert isinstance(cfg, lb.KirenexConfig)
    folder = lb.write_model_folder(cfg, tmp_path / "m", seed=3)
    arch, again = load_config(folder)
    assert again == cfg
    from safetensors.torch import load_file

    stored = load_file(str(folder / "model.safetensors"))
    assert set(stored) == {s.name for s in spec_for_config(cfg).tensor_specs()}
    assert stored["pos"].shape == (cfg.max_positions, cfg.width) and "l2.mix.dkv" not in stored
