"""Hugging Face checkpoint loading without the ``transformers`` package: our AutoModel against transformers' own
modules on the same saved directory (transformers is only the oracle here), the safetensors reader, the tokenizers."""
import json
import os

import pytest
import torch

from prometorch_b200.io.safetensors import SafeTensorsFile, load_file, load_index, save_file
from prometorch_b200.transformers_compat import AutoModel, AutoTokenizer, _detect_architecture

transformers = pytest.importorskip("transformers")


def _save(model, d):
    model.eval()
    model.save_pretrained(str(d))
    return str(d)


def _ids(vocab, B=2, T=11, seed=0):
    return torch.randint(0, vocab, (B, T), generator=torch.Generator().manual_seed(seed))


def test_bert_matches_transformers(tmp_path):
    cfg = transformers.BertConfig(vocab_size=120, hidden_size=48, num_hidden_layers=2, num_attention_heads=4, intermediate_size=96,
                                  max_position_embeddings=64, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    torch.manual_seed(0)
    ref = transformers.BertModel(cfg)
    d = _save(ref, tmp_path)
    ours = AutoModel.from_pretrained(d)
    ids = _ids(120)
    tt = torch.randint(0, 2, ids.shape, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = ref(input_ids=ids, token_type_ids=tt).last_hidden_state
        got = ours(ids, tt)
    assert type(ours).__name__ == "BertModel" and torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())


def test_gpt2_matches_transformers(tmp_path):
    cfg = transformers.GPT2Config(vocab_size=130, n_embd=48, n_layer=2, n_head=4, n_positions=64, resid_pdrop=0.0, embd_pdrop=0.0,
                                  attn_pdrop=0.0)
    torch.manual_seed(1)
    ref = transformers.GPT2LMHeadModel(cfg)                      # weights carry the "transformer." prefix
    d = _save(ref, tmp_path)
    ours = AutoModel.from_pretrained(d)
    ids = _ids(130, seed=2)
    with torch.no_grad():
        want = ref.transformer(input_ids=ids).last_hidden_state
        got = ours(ids)
    assert type(ours).__name__ == "GPT2Model" and torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())


def test_llama_matches_transformers_and_engine_loads_it(tmp_path):
    cfg = transformers.LlamaConfig(vocab_size=140, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                   intermediate_size=96, max_position_embeddings=128, rms_norm_eps=1e-5, tie_word_embeddings=False)
    torch.manual_seed(2)
    ref = transformers.LlamaForCausalLM(cfg)
    d = _save(ref, tmp_path)
    ours = AutoModel.from_pretrained(d)
    ids = _ids(140, seed=3)
    with torch.no_grad():
        want = ref.model(input_ids=ids).last_hidden_state
        got = ours(ids)
    assert type(ours).__name__ == "LlamaModel" and torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())
    # the paged engine reads the same directory and its greedy continuation equals transformers' own
    from prometorch_b200.serve.llm import GenerationConfig, LLMEngine
    eng = LLMEngine(device="cpu", max_pages=8, max_active=1)
    assert eng.load(d)
    prompt = [1, 17, 93, 4, 55]
    r = eng.generate(prompt, GenerationConfig(max_new_tokens=6, temperature=0.0, repetition_penalty=1.0, top_k=1))
    with torch.no_grad():
        out = ref.generate(torch.tensor([prompt]), max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(prompt):].tolist()
    eos = eng.cfg.eos_token_id
    want_ids = out[:out.index(eos) + 1] if eos in out else out
    assert r.token_ids == want_ids


def test_architecture_detection_and_errors(tmp_path):
    assert _detect_architecture({"architectures": ["LlamaForCausalLM"]}) == "LlamaForCausalLM"
    assert _detect_architecture({"model_type": "gpt2"}) == "GPT2Model"
    with pytest.raises(ValueError):
        _detect_architecture({"model_type": "mamba"})
    with pytest.raises(FileNotFoundError):
        AutoModel.from_pretrained(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "bert", "hidden_size": 8, "num_attention_heads": 2,
                                                      "intermediate_size": 8, "vocab_size": 9, "num_hidden_layers": 1}))
    with pytest.raises(FileNotFoundError):
        AutoModel.from_pretrained(str(tmp_path))                 # a config but no weights


def test_safetensors_file_api_and_index(tmp_path):
    a = {"x": torch.randn(4, 3), "y": torch.arange(5, dtype=torch.int32)}
    b = {"z": torch.randn(2, 2).bfloat16()}
    save_file(a, str(tmp_path / "s1.safetensors"), metadata={"format": "pt"})
    save_file(b, str(tmp_path / "s2.safetensors"))
    with SafeTensorsFile(str(tmp_path / "s1.safetensors")) as f:
        assert sorted(f.keys()) == ["x", "y"] and "x" in f and len(f) == 2 and f.metadata == {"format": "pt"}
        assert f.info("x")["shape"] == [4, 3] and torch.equal(f.get_tensor("y"), a["y"])
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "s1.safetensors", "y": "s1.safetensors", "z": "s2.safetensors"}}))
    got = load_index(str(tmp_path / "model.safetensors.index.json"))
    assert set(got) == {"x", "y", "z"} and torch.equal(got["z"], b["z"]) and torch.equal(load_file(str(tmp_path / "s1.safetensors"))["x"], a["x"])
    # the safetensors package reads what we wrote, and we read what it writes
    st = pytest.importorskip("safetensors.torch")
    assert torch.equal(st.load_file(str(tmp_path / "s2.safetensors"))["z"], b["z"])
    st.save_file({"w": torch.ones(3, dtype=torch.float16)}, str(tmp_path / "theirs.safetensors"))
    assert torch.equal(load_file(str(tmp_path / "theirs.safetensors"))["w"], torch.ones(3, dtype=torch.float16))
    (tmp_path / "bad.safetensors").write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(ValueError):
        SafeTensorsFile(str(tmp_path / "bad.safetensors"))


def test_tokenizers(tmp_path):
    wp = tmp_path / "wp"
    wp.mkdir()
    (wp / "vocab.txt").write_text("\n".join(["[PAD]", "[UNK]", "hello", "world", "##s", "!", "un", "##known"]) + "\n")
    tok = AutoTokenizer.from_pretrained(str(wp))
    ids = tok.encode("Hello worlds! zzz")
    assert ids == [2, 3, 4, 5, 1] and tok.decode(ids[:4]) == "hello worlds !"
    bpe = tmp_path / "bpe"
    bpe.mkdir()
    from prometorch_b200.io.tokenizer import _bytes_to_unicode
    b2u = _bytes_to_unicode()
    base = [b2u[b] for b in range(256)]
    vocab = {t: i for i, t in enumerate(base)}
    merges = ["h e", "he l", "hel l", "hell o"]
    for m in merges:
        vocab["".join(m.split())] = len(vocab)
    (bpe / "vocab.json").write_text(json.dumps(vocab))
    (bpe / "merges.txt").write_text("#version: 0.2\n" + "\n".join(merges) + "\n")
    tok = AutoTokenizer.from_pretrained(str(bpe))
    ids = tok.encode("hello")
    assert ids == [vocab["hello"]] and tok.decode(ids) == "hello"
    with pytest.raises(FileNotFoundError):
        AutoTokenizer.from_pretrained(str(tmp_path / "nothing"))


def test_model_loader_sniffs_and_describes_every_container(tmp_path):
    """detect_format by content, tensor metadata, inferred architecture / shape parameters, lazy tensor reads."""
    from prometorch_b200 import serialization
    from prometorch_b200.io.model_loader import detect_format, find_shard_files, infer_architecture, load_model, read_tensor
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    from prometorch_b200.serve.llm import LlamaConfig, LlamaWeights
    cfg = LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=256)
    sd = LlamaWeights.random(cfg, seed=1).state_dict()
    st = str(tmp_path / "weights.bin")                      # wrong extension on purpose: content decides
    save_file(sd, st)
    pt, ptor = str(tmp_path / "m.safetensors.pt"), str(tmp_path / "m.ptor")
    serialization.save_pytorch(dict(sd), pt)
    serialization.save_state_dict(dict(sd), ptor)
    gg = str(tmp_path / "tiny.gguf")
    write_synthetic_gguf(gg, tiny_qwen3_config(), seed=0)
    assert [detect_format(p) for p in (st, pt, ptor, gg)] == ["safetensors", "pytorch", "ptor", "gguf"]
    (tmp_path / "junk.dat").write_bytes(b"\\x00\\x01\\x02\\x03 not a model")
    assert detect_format(str(tmp_path / "junk.dat")) == "unknown" and detect_format(str(tmp_path / "missing")) == "unknown"
    for path in (st, pt, ptor):
        mw = load_model(path)
        assert mw.architecture == "llama" and len(mw.tensors) == len(sd) and mw.total_parameters() == sum(t.numel() for t in sd.values())
        c = mw.config
        assert (c.vocab_size, c.hidden_size, c.num_layers, c.intermediate_size) == (300, 64, 2, 96) and not c.tie_word_embeddings
        assert torch.equal(read_tensor(mw, "model.norm.weight"), sd["model.norm.weight"])
    g = load_model(gg)
    assert g.format == "gguf" and g.architecture == "qwen3" and g.config.num_layers >= 1 and g.config.num_heads >= 1
    assert read_tensor(g, "token_embd.weight").shape[1] == g.config.hidden_size
    # a Hugging Face directory with two shards and a config
    d = tmp_path / "hf"
    d.mkdir()
    names = sorted(sd)
    save_file({k: sd[k] for k in names[:7]}, str(d / "model-00001-of-00002.safetensors"))
    save_file({k: sd[k] for k in names[7:]}, str(d / "model-00002-of-00002.safetensors"))
    (d / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {k: f"model-0000{1 if i < 7 else 2}-of-00002.safetensors" for i, k in enumerate(names)}}))
    (d / "config.json").write_text(json.dumps({"model_type": "llama", "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
                                               "num_key_value_heads": 2, "intermediate_size": 96, "vocab_size": 300, "rope_theta": 5e5,
                                               "max_position_embeddings": 256}))
    assert detect_format(str(d)) == "hf_dir" and len(find_shard_files(str(d))) == 2
    h = load_model(str(d))
    assert h.architecture == "llama" and len(h.tensors) == len(sd) and h.config.num_kv_heads == 2 and h.config.head_dim == 16
    assert h.config.rope_freq_base == 5e5 and h.config.context_length == 256
    assert torch.equal(read_tensor(h, names[-1]), sd[names[-1]])
    assert infer_architecture(["bert.encoder.layer.0.attention.self.query.weight"]) == "bert"
    assert infer_architecture(["transformer.h.0.attn.c_attn.weight"]) == "gpt2"
    with pytest.raises(ValueError):
        load_model(str(tmp_path / "junk.dat"))


def test_legacy_pytorch_model_bin_directory(tmp_path):
    """A directory that only has ``pytorch_model.bin`` (written by torch.save) loads through the restricted .pt reader."""
    from prometorch_b200.io.model_loader import load_model
    cfg = transformers.GPT2Config(vocab_size=90, n_embd=32, n_layer=1, n_head=2, n_positions=32, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    torch.manual_seed(4)
    ref = transformers.GPT2Model(cfg).eval()
    d = tmp_path / "legacy"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg.to_dict()))
    torch.save({k: v.clone() for k, v in ref.state_dict().items()}, str(d / "pytorch_model.bin"))
    ours = AutoModel.from_pretrained(str(d))
    ids = _ids(90, T=9, seed=6)
    with torch.no_grad():
        assert torch.allclose(ours(ids), ref(input_ids=ids).last_hidden_state, atol=2e-5)
    mw = load_model(str(d))
    assert mw.architecture == "gpt2" and mw.config.num_layers == 1 and mw.config.hidden_size == 32 and mw.format == "pytorch"
