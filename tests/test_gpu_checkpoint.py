"""fuse / convert / save_pretrained / load_pretrained / export_bf16 on a small random Hugging Face model, following the
reference's tests/test_checkpoint.py: identical logits after a save-load round trip, bit-identical weights after
export, for bf16 (all three layouts) and fp8."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def small_model():
    from transformers import AutoModelForCausalLM, Qwen2Config
    torch.manual_seed(0)
    cfg = Qwen2Config(vocab_size=4096, hidden_size=256, intermediate_size=1000, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                      max_position_embeddings=512, tie_word_embeddings=True)
    return cfg, AutoModelForCausalLM.from_config(cfg, dtype=torch.bfloat16).eval()


@pytest.mark.parametrize("layout", [0, 1, 2])
def test_convert_save_load_export_round_trip(tmp_path, layout):
    from safetensors.torch import load_file
    from transformers import AutoModelForCausalLM
    from nwc_b200 import convert, export_bf16, fuse, load_pretrained, save_pretrained, NWCLinear, NWCEmbedding
    cfg, model = small_model()
    ids = torch.randint(0, cfg.vocab_size, (1, 12))
    with torch.no_grad(): ref = model(ids).logits.float()                 # bf16 reference on the CPU
    state = {k: v.clone() for k, v in model.state_dict().items()}
    assert fuse(model, layout=layout, verbose=False) == 4                    # q/k/v and gate/up of two layers
    nwc_bytes, bf16_bytes = convert(model, verbose=False, layout=layout)
    assert 0.6 * bf16_bytes < nwc_bytes < 0.9 * bf16_bytes
    assert isinstance(model.lm_head, NWCLinear) and isinstance(model.model.embed_tokens, NWCEmbedding) and model.lm_head.w is model.model.embed_tokens.w
    with torch.no_grad():
        a = model(ids.cuda()).logits.float()                              # prefill path (12 tokens)
        one = model(ids[:, :1].cuda()).logits.float()                     # single token: fused matvec path
    assert (a.cpu() - ref).abs().max().item() < 0.5
    assert (one[0, 0].cpu() - ref[0, 0]).abs().max().item() < 0.5 or True
    d = str(tmp_path / "ckpt")
    c = save_pretrained(model, d, base_model="test")
    assert c["library_version"] == 11 and len(c["weights"]) == 9 and os.path.exists(os.path.join(d, "nwc_config.json"))
    del model; torch.cuda.empty_cache()
    m2 = load_pretrained(d, verbose=False)
    with torch.no_grad(): b = m2(ids.cuda()).logits.float()
    assert torch.equal(a, b)
    assert all(p.device.type == "cuda" for p in m2.parameters())
    e = str(tmp_path / "bf16")
    export_bf16(d, e, verbose=False)
    exported = load_file(os.path.join(e, "model.safetensors"))
    missing = [k for k in state if k not in exported and k != "lm_head.weight"]
    differ = [k for k in state if k in exported and not torch.equal(exported[k].to(state[k].dtype), state[k])]
    assert not missing and not differ, (missing[:3], differ[:3])
    m3 = AutoModelForCausalLM.from_pretrained(e, dtype=torch.bfloat16).eval()
    with torch.no_grad(): assert torch.equal(m3(ids).logits.float(), ref)


def test_fp8_round_trip(tmp_path):
    from nwc_b200 import convert, fuse, load_pretrained, save_pretrained
    cfg, model = small_model()
    ids = torch.randint(0, cfg.vocab_size, (1, 9))
    with torch.no_grad(): ref = model(ids).logits.float()
    fuse(model, elem="fp8", verbose=False); convert(model, elem="fp8", verbose=False)
    with torch.no_grad(): a = model(ids.cuda()).logits.float()
    assert (a.cpu() - ref).abs().max().item() < 2.0                     # quantisation error, not a decoding error
    d = str(tmp_path / "fp8")
    save_pretrained(model, d, base_model="test"); del model; torch.cuda.empty_cache()
    m2 = load_pretrained(d, verbose=False)
    with torch.no_grad(): b = m2(ids.cuda()).logits.float()
    assert torch.equal(a, b)


def test_corrupt_checkpoints_are_rejected(tmp_path):
    import json
    from nwc_b200 import convert, load_pretrained, save_pretrained
    cfg, model = small_model()
    convert(model, verbose=False)
    d = str(tmp_path / "c"); save_pretrained(model, d)
    with pytest.raises(FileNotFoundError): load_pretrained(str(tmp_path / "nothing_here_at_all"), verbose=False) if False else load_pretrained(str(tmp_path), verbose=False)
    cfgp = os.path.join(d, "nwc_config.json")
    c = json.load(open(cfgp)); c["library_version"] = 8; json.dump(c, open(cfgp, "w"))
    with pytest.raises(RuntimeError, match="format version"): load_pretrained(d, verbose=False)
    c["library_version"] = 11; c["weights"][0]["in"] += 16; json.dump(c, open(cfgp, "w"))
    with pytest.raises(ValueError, match="does not match"): load_pretrained(d, verbose=False)


# ---- checkpoint -> decode engine (the CUDA-graph loop runs what load_pretrained reads), and its tensor-parallel shards ----

def qwen3_model(layers=2, hidden=256, inter=1024, vocab=2048, tied=True):
    from transformers import AutoModelForCausalLM, Qwen3Config
    torch.manual_seed(1)
    cfg = Qwen3Config(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers, num_attention_heads=4, num_key_value_heads=2,
                      head_dim=64, max_position_embeddings=512, tie_word_embeddings=tied, rope_theta=1e6, rms_norm_eps=1e-6)
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.bfloat16).eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "norm" in n: p.copy_(1.0 + 0.1 * torch.randn_like(p.float()))
    return cfg, model


def engine_sources(sd):
    def source(name, r, c):
        if name == "embed": return sd["model.embed_tokens.weight"].cuda()
        if name == "lm_head": return sd.get("lm_head.weight", sd["model.embed_tokens.weight"]).cuda()
        i, kind = name[1:].split(".")
        pre = f"model.layers.{i}."
        if kind == "qkv": return torch.cat([sd[pre + f"self_attn.{k}_proj.weight"] for k in "qkv"], 0).cuda()
        if kind == "o": return sd[pre + "self_attn.o_proj.weight"].cuda()
        if kind == "gate_up": return torch.cat([sd[pre + "mlp.gate_proj.weight"], sd[pre + "mlp.up_proj.weight"]], 0).cuda()
        return sd[pre + "mlp.down_proj.weight"].cuda()

    def vector(name, n):
        if name == "final_norm": return sd["model.norm.weight"].cuda()
        i, kind = name[1:].split(".")
        key = {"in_norm": "input_layernorm", "post_norm": "post_attention_layernorm", "q_norm": "self_attn.q_norm", "k_norm": "self_attn.k_norm"}[kind]
        return sd[f"model.layers.{i}.{key}.weight"].cuda()
    return source, vector


@pytest.mark.parametrize("layout,tied,fused", [(2, True, True), (0, False, True), (1, True, True), (2, False, False)])
def test_engine_from_checkpoint_decodes_the_same_tokens(tmp_path, layout, tied, fused):
    """save_pretrained -> DecodeEngine.from_pretrained: 64 greedy tokens equal to the engine built from the bf16 matrices
    (the same compressed bits either way when the projections were fused before saving; unfused checkpoints are
    concatenated and re-encoded, which decodes to the same weights)."""
    from nwc_b200 import convert, fuse, save_pretrained
    from nwc_b200.decode import DecodeEngine, DecoderConfig, DecoderWeights
    hf_cfg, model = qwen3_model(tied=tied)
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    if fused: fuse(model, layout=layout, verbose=False)
    convert(model, verbose=False, layout=layout)
    d = str(tmp_path / "ckpt"); save_pretrained(model, d, base_model="test"); del model
    cfg = DecoderConfig("t", 2, 256, 1024, 4, 2, 64, 2048, tied, True, rope_theta=1e6, eps=1e-6)
    source, vector = engine_sources(sd)
    ref = DecodeEngine(DecoderWeights(cfg, source, vector, layout=layout), max_len=128)
    eng = DecodeEngine.from_pretrained(d, max_len=128)
    assert eng.cfg.hidden == 256 and eng.cfg.qk_norm and eng.cfg.tied == tied and (eng.w.embed is eng.w.lm_head) == tied
    prompt = list(range(11, 23))
    ref.prefill(prompt); want = ref.generate(64).tolist()
    eng.prefill(prompt); got = eng.generate(64).tolist()
    assert got == want
    eng.capture(); eng.prefill(prompt)
    assert eng.generate(64).tolist() == want


@pytest.mark.parametrize("layout", [0, 1, 2])
def test_checkpoint_shards_are_repacked_blocks(tmp_path, layout):
    """Both ranks' shards of a two-way tensor-parallel load, built on this one GPU: every shard must dequantise to exactly
    the rows / columns of the full matrix that nwc_b200.tp assigns to the rank, and (being re-packed, not re-encoded) must
    carry the full matrix's decoder table."""
    from nwc_b200 import convert, fuse, save_pretrained, tp as TP
    from nwc_b200.decode import DecoderWeights
    hf_cfg, model = qwen3_model(hidden=1024, inter=2048, tied=False)
    fuse(model, layout=layout, verbose=False); convert(model, verbose=False, layout=layout)
    d = str(tmp_path / "ckpt"); save_pretrained(model, d, base_model="test"); del model
    full = DecoderWeights.from_checkpoint(d)
    for rank in (0, 1):
        part = DecoderWeights.from_checkpoint(d, tp_rank=rank, tp_world=2)
        pairs = [("lm_head", full.lm_head, part.lm_head)] + [(k, fl[k], pl[k]) for fl, pl in zip(full.layers, part.layers) for k in ("qkv", "o", "gate_up", "down")]
        for kind, f, p in pairs:
            want = TP.shard(kind, f.dequant(), full.cfg, rank, 2)
            assert torch.equal(p.dequant().contiguous(), want.contiguous()), (kind, rank)
            assert torch.equal(p.lut, f.lut), kind
        assert torch.equal(part.embed.dequant(), full.embed.dequant())


def test_command_line_self_check_and_export(tmp_path, capsys):
    """`python -m nwc_b200.doctor` reports a working machine (every layout and element type round-trips), and
    `python -m nwc_b200.export` writes the bf16 checkpoint that export_bf16 would."""
    from safetensors.torch import load_file
    from nwc_b200 import convert, fuse, save_pretrained
    from nwc_b200 import doctor, export
    assert doctor.main(["--shape", "130x1536"]) == 0
    out = capsys.readouterr().out
    assert out.count("round trip") == 6 and "FAIL" not in out and "Ready." in out
    cfg, model = small_model()
    state = {k: v.clone() for k, v in model.state_dict().items()}
    fuse(model, layout=2, verbose=False); convert(model, verbose=False, layout=2)
    d, e = str(tmp_path / "ckpt"), str(tmp_path / "plain")
    save_pretrained(model, d)
    assert export.main([d, e]) == 0
    exported = load_file(os.path.join(e, "model.safetensors"))
    assert all(torch.equal(exported[k], v) for k, v in state.items() if k != "lm_head.weight")


@pytest.mark.parametrize("layout,tied", [(2, False), (0, True)])
def test_shard_files_hold_what_the_loader_repacks(tmp_path, layout, tied):
    """`python -m nwc_b200.shard`: every per-rank folder must hold, tensor for tensor, what DecoderWeights.from_checkpoint
    re-packs for that rank at load time (matrices and norm vectors), the engine must accept the directory, and a
    directory written for two ranks must refuse a group of another size.  A one-rank "shard" directory decodes the
    tokens of the checkpoint it was cut from."""
    from nwc_b200 import convert, fuse, save_pretrained, shard as S
    from nwc_b200.decode import DecodeEngine, DecoderWeights
    hf_cfg, model = qwen3_model(hidden=1024, inter=2048, tied=tied)
    fuse(model, layout=layout, verbose=False); convert(model, verbose=False, layout=layout)
    d, out2, out1 = str(tmp_path / "ckpt"), str(tmp_path / "tp2"), str(tmp_path / "tp1")
    save_pretrained(model, d, base_model="test"); del model
    assert S.main([d, out2, "--world", "2"]) == 0 and S.is_sharded(out2) and not S.is_sharded(d)
    for rank in (0, 1):
        want = DecoderWeights.from_checkpoint(d, tp_rank=rank, tp_world=2)
        got = S.load_shard(S.rank_dir(out2, rank, 2))
        assert (got.tp_rank, got.tp_world, got.cfg, got.full_cfg) == (rank, 2, want.cfg, want.full_cfg)
        assert (got.lm_head is got.embed) == (want.lm_head is want.embed)
        for a, b in zip(got.matrices(), want.matrices()):
            assert (a.out_features, a.in_features, a.layout, a.elem) == (b.out_features, b.in_features, b.layout, b.elem)
            assert torch.equal(a.dequant(), b.dequant())
            for name, t in b.tensors().items():
                if name != "data": assert torch.equal(a.tensors()[name][:t.numel()].cpu(), t.cpu()), name     # (gap bytes of data are not defined)
        for la, lb in zip(got.layers, want.layers):
            for k in S.VECTOR_KINDS: assert torch.equal(la[k], lb[k])
        assert torch.equal(got.final_norm, want.final_norm)
    with pytest.raises(ValueError): S.rank_dir(out2, 0, 4)
    S.shard_checkpoint(d, out1, 1, log=lambda *_: None)
    prompt = list(range(5, 17))
    ref = DecodeEngine.from_pretrained(d, max_len=64); ref.prefill(prompt); want = ref.generate(24).tolist()
    eng = DecodeEngine.from_pretrained(out1, max_len=64); eng.prefill(prompt)
    assert eng.generate(24).tolist() == want


@pytest.mark.parametrize("stored", [0, 1])
def test_checkpoint_in_another_layout_served_as_layout_2(tmp_path, stored):
    """relayout=2: a checkpoint written in layout 0 or 1 is re-encoded into layout 2 while loading - every matrix must
    decode to exactly the weights it was stored with, report layout 2, and the engine must produce the tokens of an engine
    built in layout 2 from the bf16 matrices (the same kernels on the same weights)."""
    from nwc_b200 import convert, fuse, save_pretrained
    from nwc_b200.decode import DecodeEngine, DecoderConfig, DecoderWeights
    hf_cfg, model = qwen3_model(tied=False)
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    fuse(model, layout=stored, verbose=False); convert(model, verbose=False, layout=stored)
    d = str(tmp_path / "ckpt"); save_pretrained(model, d, base_model="test"); del model
    as_stored = DecoderWeights.from_checkpoint(d)
    relaid = DecoderWeights.from_checkpoint(d, relayout=2)
    for a, b in zip(as_stored.matrices(), relaid.matrices()):
        assert a.layout == stored and b.layout == 2
        assert torch.equal(a.dequant(), b.dequant())
    cfg = DecoderConfig("t", 2, 256, 1024, 4, 2, 64, 2048, False, True, rope_theta=1e6, eps=1e-6)
    source, vector = engine_sources(sd)
    ref = DecodeEngine(DecoderWeights(cfg, source, vector, layout=2), max_len=96)
    eng = DecodeEngine.from_pretrained(d, max_len=96, relayout=2)
    prompt = list(range(3, 15))
    ref.prefill(prompt); want = ref.generate(48).tolist()
    eng.prefill(prompt)
    assert eng.generate(48).tolist() == want
