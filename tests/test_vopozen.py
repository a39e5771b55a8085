"""Vopozen without a device: configuration (also the size that is read from a stored tensor), the spec's tensors
and parts, and what the cache manager makes of a chunked mask, of a windowed latent that several layers read
through windows of their own, and of the recurrent layers' state rows."""

import json

import pytest
import torch

import layover_b200 as lb
from layover_b200.cache import CacheManager
from layover_b200.config.base import load_config, resolve_architecture
from layover_b200.models import assemble, spec_for_config
from layover_b200.parts.base import PagedKVNeed, StateNeed
from vopozen_configs import CONFIGS, attention, config, dense, latent, moe, wkv


@pytest.mark.parametrize("name", list(CONFIGS))
def test_config_round_trip_and_registry(name, tmp_path):
    raw = CONFIGS[name]
    cfg = lb.VopozenConfig.from_hf_dict(raw)
    assert lb.VopozenConfig.from_hf_dict(cfg.to_hf_dict()) == cfg
    assert resolve_architecture(raw).config_class is lb.VopozenConfig
    (tmp_path / "config.json").write_text(json.dumps(raw))
    arch, again = load_config(tmp_path)
    assert arch.name == "Vopozen" and again == cfg


def test_the_decay_rank_comes_from_the_stored_tensor_where_the_configuration_leaves_it_out(tmp_path):
    raw = CONFIGS["odd_sizes"]
    folder = lb.write_model_folder(lb.VopozenConfig.from_hf_dict(raw), tmp_path, seed=1)
    stripped = json.loads((folder / "config.json").read_text())
    for layer in stripped["layers"]:
        layer["mixer"].pop("decay_rank", None)
    (folder / "config.json").write_text(json.dumps(stripped))
    _, cfg = load_config(folder)
    assert cfg == lb.VopozenConfig.from_hf_dict(raw)
    assert [l["mixer"]["decay_rank"] for l in cfg.layers if l["type"] == "wkv"] == [5, 3]
    with pytest.raises(ValueError, match="decay_rank"):
        lb.VopozenConfig.from_hf_dict(stripped)           # no folder, no shapes


def test_refusals():
    good = CONFIGS["odd_sizes"]
    for change, match in [
        (lambda c: c["layers"][0].update(type="parallel"), "unknown type"),
        (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
        (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4), "rot.dims must equal rot_dim"),
        (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "earlier layer"),
        (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "latent_attention layer"),
        (lambda c: c["layers"][3]["mixer"].update(kv_rank=40), "must equal those of layer 1"),
        (lambda c: c["layers"][2]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
        (lambda c: c["layers"][2]["mixer"].update(vdim=16), "vdim must equal dim"),
        (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=14), "rot"),
        (lambda c: c["layers"][2]["mixer"]["mask"].update(size=0), "mask.size"),
        (lambda c: c["layers"][2]["mixer"].update(scale=0), "scale"),
        (lambda c: c["layers"][0]["mixer"].update(heads=0), "heads"),
        (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "mlp kind"),
        (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "exceeds the experts"),
        (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "do not fit"),
        (lambda c: c["layers"][5]["mlp"]["router"]["groups"].update(keep=1), "fewer experts than a token chooses"),
        (lambda c: c.update(residual_mult=0.0), "residual_mult"),
        (lambda c: c.pop("width"), "lacks"),
    ]:
        raw = json.loads(json.dumps(good))
        change(raw)
        with pytest.raises(ValueError, match=match):
            lb.VopozenConfig.from_hf_dict(raw)


def test_the_specs_tensors_have_the_checkpoints_names_and_shapes():
    raw = config(50, 24, [
        wkv(3, 4, 5, dense(14)),
        attention(4, 2, 8, 5, 4, 100.0, 0.1, mlp=moe(3, 2, 6, 1.5, shared=10)),
        latent(3, 4, 2, 6, 10, 7, 100.0, 0.3),
        latent(2, 8, 2, 4, 10, 9, 100.0, 0.2, kv_from=2, mlp=dense(18)),
    ], mult=0.5)
    spec = spec_for_config(lb.VopozenConfig.from_hf_dict(raw))
    shapes = {s.name: tuple(s.shape) for s in spec.tensor_specs()}
    assert shapes == {
        "embed": (50, 24), "final.norm": (24,), "head": (50, 24),
        "l0.norm1": (24,), "l0.norm2": (24,),
        **{f"l0.mix.mu.{s}": (24,) for s in "rkvgw"},
        "l0.mix.r": (12, 24), "l0.mix.k": (12, 24), "l0.mix.v": (12, 24), "l0.mix.g": (12, 24),
        "l0.mix.w1": (5, 24), "l0.mix.w2": (12, 5), "l0.mix.w0": (12,), "l0.mix.u": (3, 4), "l0.mix.norm": (12,), "l0.mix.o": (24, 12),
        "l0.mlp.gate": (14, 24), "l0.mlp.up": (14, 24), "l0.mlp.down": (24, 14),
        "l1.norm1": (24,), "l1.norm2": (24,),
        "l1.mix.q": (32, 24), "l1.mix.k": (16, 24), "l1.mix.q.norm": (8,), "l1.mix.k.norm": (8,), "l1.mix.o": (24, 32),
        "l1.mlp.router": (3, 24), "l1.mlp.correction": (3,),
        **{f"l1.mlp.e{e}.up": (6, 24) for e in range(3)}, **{f"l1.mlp.e{e}.down": (24, 6) for e in range(3)},
        "l1.mlp.shared.up": (10, 24), "l1.mlp.shared.down": (24, 10),
        "l2.norm1": (24,),
        "l2.mix.q": (18, 24), "l2.mix.dkv": (12, 24), "l2.mix.dkv.norm": (10,), "l2.mix.uk": (12, 10), "l2.mix.uv": (18, 10), "l2.mix.o": (24, 18),
        "l3.norm1": (24,), "l3.norm2": (24,),
        "l3.mix.q": (20, 24), "l3.mix.uk": (16, 10), "l3.mix.uv": (8, 10), "l3.mix.o": (24, 8),
        "l3.mlp.gate": (18, 24), "l3.mlp.up": (18, 24), "l3.mlp.down": (24, 18),
    }
    assert spec.ignorable_tensors == {"l2.norm2"} and spec.residual_dtype == "float32"
    assert [e.reads_cache_of for e in spec.schedule] == [None, None, None, 2]
    kinds = {s.name: s.kind for s in spec.tensor_specs()}
    assert kinds["l1.mlp.router"] == "keep32" and kinds["l1.mlp.correction"] == "keep32" and kinds["l0.mix.w0"] == "vector"


def test_cache_groups_a_shared_latent_keeps_the_widest_window_and_state_rows_hold_the_previous_input():
    cfg = lb.VopozenConfig.from_hf_dict(CONFIGS["odd_sizes"])
    model = assemble(spec_for_config(cfg), cfg)
    needs = model.cache_needs()
    # the latent of layer 1 (window 9) is read by layer 3 through a window of 33: its rows are kept for 33 tokens
    assert needs[1][1] == PagedKVNeed(1, 44, window=33, values_in_keys=True) and needs[3][2] == 1
    assert needs[2][1] == PagedKVNeed(2, 12, chunk=24) and needs[5][1] == PagedKVNeed(1, 24, chunk=7)
    assert needs[0][1] == StateNeed((3 * 12 * 12 + 72,), torch.float32) and needs[4][1] == StateNeed((2 * 20 * 20 + 72,), torch.float32)
    cache = CacheManager(needs, 64, 4, torch.float32, None, 4)
    assert len(cache.paged) == 3 and len(cache.states) == 2
    assert cache.views[3].group == cache.views[1].group and not cache.views[3].writes
    seq = cache.open("a")
    cache.grow(seq, 100)
    cache.commit(seq, 100)
    tables = dict(zip((g.need for g in cache.paged), seq.tables))
    windowed = tables[needs[1][1]]
    assert windowed.first_live == (100 - 33 + 1) // 4          # the pages the widest window has passed went back
    chunked = tables[needs[2][1]]
    assert chunked.first_live == (100 // 24 * 24) // 4         # and the pages of finished chunks
    cache.close(seq)
    cache.check()


def test_a_reader_with_a_narrower_window_does_not_shrink_what_the_writer_keeps():
    cfg = lb.VopozenConfig.from_hf_dict(CONFIGS["wide_heads"])
    needs = assemble(spec_for_config(cfg), cfg).cache_needs()
    assert needs[1][1].window == 40 and needs[2][2] == 1 and needs[6][2] == 1      # windows 24 (own), 5 and 40 (readers)
    blocks = {b.mixer.window for b in assemble(spec_for_config(cfg), cfg).blocks if hasattr(b.mixer, "cache_window")}
    assert blocks == {24, 5, 40}


def test_preset():
    cfg = lb.preset("vopozen-tiny")
    assert isinstance(cfg, lb.VopozenConfig) and len(cfg.layers) == 5
    assert spec_for_config(cfg).tensor_specs()
