"""HF encoder families on CPU: numerical parity with the `transformers` implementations (tiny random
configs, weights moved through safetensors), key maps, config round trips, safetensors validation."""
import json
import os

import pytest
import torch

from flodl_b200 import hf
from flodl_b200.hf import safetensors_io as st
from flodl_b200.hf.models import albert, bert, deberta_v2, distilbert, roberta, xlm_roberta
from flodl_b200.hf.path import HfPath, hf_key_from_flodl_key

transformers = pytest.importorskip("transformers")

IDS = torch.tensor([[2, 5, 6, 7, 3, 0, 0, 0], [2, 9, 10, 11, 12, 13, 14, 3]])
PAD = 0


def hf_state_bytes(model) -> bytes:
    # like `save_pretrained`: tensors that share storage (tied weights) are written once
    sd, seen = {}, set()
    for k, v in sorted(model.state_dict().items()):
        if not v.is_floating_point() or v.data_ptr() in seen:
            continue
        seen.add(v.data_ptr())
        sd[k] = v.detach().clone().contiguous()
    return st.write_safetensors(sd)


def load_allowing_unused(graph, blob, rename=st.bert_legacy_key_rename):
    return st.load_safetensors_into_graph_with_rename_allow_unused(graph, blob, rename)


def close(a, b, tol=2e-5):
    err = (a - b).abs().max().item()
    assert err < tol, err


def test_bert_parity_backbone_and_mlm():
    hc = transformers.BertConfig(vocab_size=50, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                                 max_position_embeddings=16, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    torch.manual_seed(0)
    hf = transformers.BertForMaskedLM(hc).eval()
    cfg = bert.BertConfig.from_json_str(hc.to_json_string())
    head = bert.BertForMaskedLM.on_device(cfg)
    head.graph().set_training(False)
    unused = load_allowing_unused(head.graph(), hf_state_bytes(hf))
    assert all("position_ids" in k or k == "cls.predictions.decoder.weight" for k in unused), unused
    mask = (IDS != PAD).float()
    pos = torch.arange(8).expand(2, 8)
    tt = torch.zeros_like(IDS)
    mine = head.forward([IDS, pos, tt, bert.build_extended_attention_mask(mask)]).t
    ref = hf(input_ids=IDS, attention_mask=mask.long(), token_type_ids=tt).logits
    close(mine[mask.bool()], ref[mask.bool()], 1e-4)


def test_roberta_parity_sequence_classification():
    hc = transformers.RobertaConfig(vocab_size=50, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                                    max_position_embeddings=20, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, num_labels=3,
                                    pad_token_id=1, type_vocab_size=1)
    torch.manual_seed(1)
    hf = transformers.RobertaForSequenceClassification(hc).eval()
    cfg = roberta.RobertaConfig.from_json_str(hc.to_json_string())
    assert cfg.num_labels == 3 and cfg.pad_token_id == 1
    head = roberta.RobertaForSequenceClassification.on_device(cfg, 3)
    head.graph().set_training(False)
    load_allowing_unused(head.graph(), hf_state_bytes(hf))
    ids = IDS.clone()
    ids[ids == 0] = 1
    mask = (ids != 1).float()
    mine = head.forward([ids, torch.zeros_like(ids), bert.build_extended_attention_mask(mask)]).t
    ref = hf(input_ids=ids, attention_mask=mask.long()).logits
    close(mine, ref, 1e-4)


def test_distilbert_parity():
    hc = transformers.DistilBertConfig(vocab_size=50, dim=32, n_layers=2, n_heads=4, hidden_dim=64, max_position_embeddings=16, dropout=0.0,
                                       attention_dropout=0.0)
    torch.manual_seed(2)
    hf = transformers.DistilBertModel(hc).eval()
    cfg = distilbert.DistilBertConfig.from_json_str(hc.to_json_string())
    g = distilbert.DistilBertModel.build(cfg)
    g.set_training(False)
    load_allowing_unused(g, hf_state_bytes(hf), lambda k: "distilbert." + k)
    mask = (IDS != PAD).float()
    mine = g.forward([IDS, bert.build_extended_attention_mask(mask)]).t
    ref = hf(input_ids=IDS, attention_mask=mask.long()).last_hidden_state
    close(mine[mask.bool()], ref[mask.bool()], 1e-4)


def test_albert_parity():
    hc = transformers.AlbertConfig(vocab_size=50, embedding_size=16, hidden_size=32, num_hidden_layers=3, num_attention_heads=4,
                                   intermediate_size=64, max_position_embeddings=16, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    torch.manual_seed(3)
    hf = transformers.AlbertModel(hc).eval()
    cfg = albert.AlbertConfig.from_json_str(hc.to_json_string())
    g = albert.AlbertModel.build(cfg)
    g.set_training(False)
    load_allowing_unused(g, hf_state_bytes(hf), lambda k: "albert." + k)
    mask = (IDS != PAD).float()
    pos = torch.arange(8).expand(2, 8)
    mine = g.forward([IDS, pos, torch.zeros_like(IDS), bert.build_extended_attention_mask(mask)]).t
    ref = hf(input_ids=IDS, attention_mask=mask.long()).pooler_output
    close(mine, ref, 1e-4)


def test_deberta_v2_parity():
    hc = transformers.DebertaV2Config(vocab_size=50, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                                      max_position_embeddings=16, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
                                      relative_attention=True, position_buckets=4, max_relative_positions=8, share_att_key=True,
                                      pos_att_type=["p2c", "c2p"], norm_rel_ebd="layer_norm", position_biased_input=False, type_vocab_size=0)
    torch.manual_seed(4)
    hf = transformers.DebertaV2Model(hc).eval()
    cfg = deberta_v2.DebertaV2Config.from_json_str(hc.to_json_string())
    g = deberta_v2.DebertaV2Model.build(cfg)
    g.set_training(False)
    load_allowing_unused(g, hf_state_bytes(hf), lambda k: "deberta." + k)
    mask = (IDS != PAD).float()
    mine = g.forward([IDS, mask]).t
    ref = hf(input_ids=IDS, attention_mask=mask.long()).last_hidden_state
    close(mine[mask.bool()], ref[mask.bool()], 1e-4)


def test_deberta_rejects_unsupported_configs():
    base = json.loads(deberta_v2.DebertaV2Config().to_json_str())
    for key, val in (("relative_attention", False), ("share_att_key", False), ("position_biased_input", True), ("pos_att_type", ["c2p"])):
        bad = dict(base)
        bad[key] = val
        with pytest.raises(Exception):
            deberta_v2.DebertaV2Config.from_json_str(json.dumps(bad))


def test_bert_key_map_matches_hf_names():
    cfg = bert.BertConfig(vocab_size=30, hidden_size=16, num_hidden_layers=1, num_attention_heads=2, intermediate_size=32, max_position_embeddings=8)
    g = bert.BertModel.build(cfg)
    keys = {e.key for e in st.expected_from_graph(g)}
    assert "bert.embeddings.word_embeddings.weight" in keys and "bert.embeddings.LayerNorm.bias" in keys
    assert "bert.encoder.layer.0.attention.self.query.weight" in keys and "bert.encoder.layer.0.output.LayerNorm.weight" in keys
    assert "bert.pooler.dense.bias" in keys and len(keys) == 5 + 16 + 2
    assert hf_key_from_flodl_key("bert.encoder.layer.0/attention.self.query.weight") == "bert.encoder.layer.0.attention.self.query.weight"
    assert str(HfPath("bert").sub("encoder").sub("layer").sub(3)) == "bert.encoder.layer.3"
    with pytest.raises(Exception):
        HfPath("a.b")


def test_config_round_trips_and_presets():
    for cfg in (bert.BertConfig.bert_base_uncased(), roberta.RobertaConfig.roberta_base(), xlm_roberta.XlmRobertaConfig.xlm_roberta_base(),
                distilbert.DistilBertConfig.distilbert_base_uncased(), albert.AlbertConfig.albert_base_v2(),
                deberta_v2.DebertaV2Config.deberta_v3_base()):
        s = cfg.to_json_str()
        assert type(cfg).from_json_str(s).to_json_str() == s
        assert json.loads(s)["model_type"] == cfg.MODEL_TYPE
    c = bert.BertConfig.from_json_str(json.dumps({**json.loads(bert.BertConfig().to_json_str()), "id2label": {"0": "neg", "1": "pos"}}))
    assert c.num_labels == 2 and c.id2label == ["neg", "pos"]
    with pytest.raises(Exception):
        bert.BertConfig.from_json_str("{}")
    with pytest.raises(Exception):
        albert.AlbertConfig.from_json_str(json.dumps({**json.loads(albert.AlbertConfig().to_json_str()), "num_hidden_groups": 2}))


def test_safetensors_validation_reports_everything_and_commits_nothing():
    cfg = bert.BertConfig(vocab_size=30, hidden_size=16, num_hidden_layers=1, num_attention_heads=2, intermediate_size=32, max_position_embeddings=8)
    g = bert.BertModel.build(cfg)
    before = [p.t.detach().clone() for p in g.parameters()]
    tensors = st.read_safetensors(st.save_safetensors_from_graph(g))
    tensors = {k: torch.zeros_like(v) for k, v in tensors.items()}
    del tensors["bert.pooler.dense.bias"]
    tensors["bert.pooler.dense.weight"] = torch.zeros(3, 3)
    tensors["extra.key"] = torch.zeros(1)
    with pytest.raises(Exception) as e:
        st.load_safetensors_into_graph(g, st.write_safetensors(tensors))
    msg = str(e.value)
    assert "missing" in msg and "bert.pooler.dense.bias" in msg and "unused" in msg and "extra.key" in msg and "shape mismatch" in msg
    assert all(torch.equal(a, p.t) for a, p in zip(before, g.parameters()))
    v = st.validate_keys([st.ExpectedParam("a", [2])], {"a": [2], "b": [1]})
    assert v.unused == ["b"] and not v.missing
    v.into_result_allow_unused()
    with pytest.raises(Exception):
        v.into_result()


def test_safetensors_format_interoperates_with_the_reference_package():
    sft = pytest.importorskip("safetensors.torch")
    t = {"w": torch.randn(3, 4), "h": torch.randn(5).half(), "b": torch.randn(2, 2).bfloat16(), "d": torch.randn(2).double()}
    mine = st.write_safetensors(t)
    theirs = sft.load(mine)
    assert all(torch.equal(t[k], theirs[k]) for k in t)
    back = st.read_safetensors(sft.save(t))
    assert all(torch.equal(t[k], back[k]) for k in t)
    with pytest.raises(Exception):
        st.write_safetensors({"i": torch.arange(3)})
    with pytest.raises(Exception):
        st.read_safetensors(sft.save({"i": torch.arange(3)}))
    with pytest.raises(Exception):
        st.parse_header(b"\x00\x01")


def test_legacy_renames_and_pooler_detection():
    assert st.bert_legacy_key_rename("bert.embeddings.LayerNorm.gamma") == "bert.embeddings.LayerNorm.weight"
    assert st.bert_legacy_key_rename("x.LayerNorm.beta") == "x.LayerNorm.bias"
    assert st.bert_legacy_key_rename("cls.predictions.bias") == "cls.predictions.decoder.bias"
    assert st.hf_canonical_save_key("lm_head.decoder.bias") == "lm_head.bias"
    assert st.keys_have_pooler(["bert.pooler.dense.weight"]) and st.keys_have_pooler(["albert/pooler.weight"])
    assert not st.keys_have_pooler(["bert.encoder.layer.0.output.dense.weight"])
    blob = st.write_safetensors({"a.LayerNorm.gamma": torch.zeros(1), "a.LayerNorm.weight": torch.zeros(1)})

    class G:
        def named_parameters(self): return []
        def named_buffers(self): return []
    with pytest.raises(Exception) as e:
        st.load_safetensors_into_graph_with_rename(G(), blob, st.bert_legacy_key_rename)
    assert "collision" in str(e.value)


def test_task_heads_losses_and_predictions():
    cfg = bert.BertConfig(vocab_size=30, hidden_size=16, num_hidden_layers=1, num_attention_heads=2, intermediate_size=32,
                          max_position_embeddings=8, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, id2label=["a", "b", "c"])
    ids = torch.randint(1, 30, (2, 8))
    inputs = [ids, torch.arange(8).expand(2, 8), torch.zeros_like(ids), bert.build_extended_attention_mask(torch.ones(2, 8))]
    clf = bert.BertForSequenceClassification.on_device(cfg, 3)
    clf.graph().set_training(False)
    loss = clf.compute_loss(inputs, torch.tensor([0, 2]))
    loss.backward()
    assert loss.t.dim() == 0 and clf.labels() == ["a", "b", "c"]
    preds = clf.predict(inputs)
    assert len(preds) == 2 and preds[0][0][0] in ("a", "b", "c")
    tag = bert.BertForTokenClassification.on_device(cfg, 3)
    assert tag.compute_loss(inputs, torch.randint(0, 3, (2, 8))).t.dim() == 0
    qa = bert.BertForQuestionAnswering.on_device(cfg)
    assert qa.compute_loss(inputs, torch.tensor([1, 2]), torch.tensor([3, 4])).t.dim() == 0
    mlm = bert.BertForMaskedLM.on_device(cfg)
    labels = torch.full((2, 8), -100)
    labels[:, 2] = ids[:, 2]
    assert mlm.compute_loss(inputs, labels).t.dim() == 0
    with pytest.raises(Exception):
        bert.BertForSequenceClassification.on_device(cfg, 0)


def test_auto_classes_export_and_local_from_pretrained(tmp_path, monkeypatch):
    from flodl_b200 import hf
    from flodl_b200.hf.export import classify_architecture, parse_head
    cfg = roberta.RobertaConfig(vocab_size=40, hidden_size=16, num_hidden_layers=1, num_attention_heads=2, intermediate_size=32,
                                max_position_embeddings=12, id2label=["no", "yes"])
    head = roberta.RobertaForSequenceClassification.on_device(cfg, 2)
    out = str(tmp_path / "hub_home" / "flodl-converted" / "acme" / "tiny-roberta")
    hf.export_hf_dir(head.graph(), head.graph().source_config(), out)
    assert sorted(p.name for p in (tmp_path / "hub_home" / "flodl-converted" / "acme" / "tiny-roberta").iterdir()) == ["config.json", "model.safetensors"]
    auto = hf.AutoConfig.from_json_str(open(out + "/config.json").read())
    assert auto.model_type() == "roberta" and auto.architectures() == ["RobertaForSequenceClassification"] and auto.base_class_name() == "RobertaModel"
    monkeypatch.setenv("HF_HOME", str(tmp_path / "hub_home"))
    g = hf.from_pretrained("acme/tiny-roberta", head="seqcls")
    for (n1, p1), (n2, p2) in zip(head.graph().named_parameters(), g.named_parameters()):
        assert n1 == n2 and torch.equal(p1.t, p2.t)
    h2 = hf.hub.sequence_classification_from_pretrained("acme/tiny-roberta")
    assert h2.labels() == ["no", "yes"]
    backbone = hf.from_pretrained("acme/tiny-roberta")            # head keys are simply unused
    assert not any(n.startswith("classifier") for n, _ in backbone.named_parameters())
    with pytest.raises(Exception) as e:
        hf.from_pretrained("acme/not-there")
    assert "not found; looked in" in str(e.value)
    assert classify_architecture("BertForMaskedLM") == "mlm" and classify_architecture("BertModel") == "base"
    assert parse_head("token-classification") == "tokcls"
    with pytest.raises(Exception):
        classify_architecture("BertForPreTraining")
    with pytest.raises(Exception):
        hf.AutoConfig.from_json_str('{"model_type": "gpt2"}')
    for mt, c in (("bert", bert.BertConfig), ("distilbert", distilbert.DistilBertConfig), ("albert", albert.AlbertConfig),
                  ("deberta-v2", deberta_v2.DebertaV2Config), ("xlm-roberta", xlm_roberta.XlmRobertaConfig)):
        assert hf.AutoConfig.from_json_str(c().to_json_str()).model_type() == mt


def test_fdl_checkpoint_exports_to_hf_dir(tmp_path):
    from flodl_b200 import hf
    cfg = bert.BertConfig(vocab_size=30, hidden_size=16, num_hidden_layers=1, num_attention_heads=2, intermediate_size=32, max_position_embeddings=8)
    g = bert.BertModel.on_device_without_pooler(cfg)
    path = str(tmp_path / "m.fdl")
    g.save_checkpoint(path)
    hf.export_checkpoint(path, str(tmp_path / "out"))
    back = st.read_safetensors(open(tmp_path / "out" / "model.safetensors", "rb").read())
    assert "bert.embeddings.word_embeddings.weight" in back and not st.keys_have_pooler(list(back))
    assert json.loads(open(tmp_path / "out" / "config.json").read())["model_type"] == "bert"


def test_tokenizer_wrapper_builds_graph_inputs(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    from flodl_b200.hf.tokenizer import HfTokenizer
    vocab = {"[PAD]": 0, "[UNK]": 1, "[CLS]": 2, "[SEP]": 3, "hello": 4, "world": 5, "again": 6}
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    tok.post_processor = tokenizers.processors.TemplateProcessing(single="[CLS] $A [SEP]", pair="[CLS] $A [SEP] $B:1 [SEP]:1",
                                                                  special_tokens=[("[CLS]", 2), ("[SEP]", 3)])
    path = str(tmp_path / "tokenizer.json")
    tok.save(path)
    t = HfTokenizer.from_file(path)
    enc = t.encode(["hello world", "hello"])
    assert enc.input_ids.tolist() == [[2, 4, 5, 3], [2, 4, 3, 0]] and enc.attention_mask.tolist() == [[1, 1, 1, 1], [1, 1, 1, 0]]
    assert enc.position_ids.tolist()[1] == [0, 1, 2, 3]
    pair = t.encode_pairs([("hello", "world again")])
    assert pair.token_type_ids.tolist() == [[0, 0, 0, 1, 1, 1]]
    ins = bert.BertConfig.encoder_inputs(enc)
    assert len(ins) == 4 and list(ins[3].t.shape) == [2, 1, 1, 4]
    assert "hello world" in t.decode([2, 4, 5, 3]) and t.token_to_id("world") == 5 and t.id_to_token(4) == "hello"
    with pytest.raises(Exception):
        t.encode([])


# ---- hub fetch, converter, parity matrix ------------------------------------------------------------------
def _serve(directory):
    """A throw-away HTTP server on 127.0.0.1 that plays the hub: GET /<repo>/resolve/<rev>/<file>."""
    import functools
    import http.server
    import threading

    class Quiet(http.server.SimpleHTTPRequestHandler):
        def log_message(self, *a):
            pass
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), functools.partial(Quiet, directory=str(directory)))
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv


def _tiny_bert_files(dst):
    hc = transformers.BertConfig(vocab_size=50, hidden_size=32, num_hidden_layers=1, num_attention_heads=4, intermediate_size=64,
                                 max_position_embeddings=16, architectures=["BertModel"])
    torch.manual_seed(0)
    hf = transformers.BertModel(hc).eval()
    dst.mkdir(parents=True, exist_ok=True)
    (dst / "config.json").write_text(hc.to_json_string())
    (dst / "model.safetensors").write_bytes(hf_state_bytes(hf))
    return hf


def test_from_pretrained_fetches_missing_files_into_the_cache_layout(tmp_path, monkeypatch):
    from flodl_b200.hf import hub
    from flodl_b200.tensor import TensorError
    _tiny_bert_files(tmp_path / "www" / "acme" / "tiny-bert" / "resolve" / "main")
    srv = _serve(tmp_path / "www")
    try:
        monkeypatch.setenv("HF_HOME", str(tmp_path / "home"))
        monkeypatch.setenv("HF_ENDPOINT", f"http://127.0.0.1:{srv.server_address[1]}")
        monkeypatch.delenv("HF_HUB_OFFLINE", raising=False)
        cfg, weights, tok = hub.resolve_files("acme/tiny-bert")
        snap = tmp_path / "home" / "hub" / "models--acme--tiny-bert" / "snapshots" / "main"
        assert cfg == str(snap / "config.json") and weights == str(snap / "model.safetensors") and tok is None
        assert not list(snap.glob("*.part"))
        g = hub.from_pretrained("acme/tiny-bert")
        assert g is not None
        # a second resolve is served from the cache: it still works with the server gone and offline mode on
        srv.shutdown()
        monkeypatch.setenv("HF_HUB_OFFLINE", "1")
        assert hub.resolve_files("acme/tiny-bert")[0] == cfg
        with pytest.raises(TensorError, match="HF_HUB_OFFLINE"):
            hub.resolve_files("acme/not-there")
        monkeypatch.delenv("HF_HUB_OFFLINE")
        with pytest.raises(TensorError, match="GET http://127.0.0.1"):
            hub.resolve_files("acme/not-there")
    finally:
        srv.shutdown()


def test_convert_bin_to_safetensors_round_trip(tmp_path, monkeypatch):
    from flodl_b200.hf import convert, hub
    src = tmp_path / "repo"
    hf = _tiny_bert_files(src)
    (src / "model.safetensors").unlink()
    torch.save(hf.state_dict(), src / "pytorch_model.bin")
    monkeypatch.setenv("HF_HOME", str(tmp_path / "home"))
    monkeypatch.setenv("HF_HUB_OFFLINE", "1")
    assert convert.main([str(src)]) == 0
    out = tmp_path / "home" / "flodl-converted" / "repo"
    back = st.read_safetensors((out / "model.safetensors").read_bytes())
    sd = hf.state_dict()
    assert set(back) == {k for k, v in sd.items()} and all(torch.equal(back[k], sd[k]) for k in back)
    assert (out / "config.json").exists()
    g = hub.from_pretrained("repo")                       # found under flodl-converted
    assert g is not None
    assert convert.main([str(tmp_path / "nothing-here")]) == 1


def test_parity_matrix_tool_covers_every_family_and_head():
    from flodl_b200.hf import parity
    res = parity.run(["bert", "distilbert"], ["base", "mlm", "qa"], "cpu", 2e-4)
    assert all(v is not None and v <= 2e-4 for v, _ in res.values()), res
    table = parity.render(res, ["bert", "distilbert"], ["base", "mlm", "qa"], 2e-4)
    assert "| bert |" in table and "FAIL" not in table and "n/a" not in table


# ---- class-level from_pretrained and the text-level head methods ------------------------------------------------
VOCAB = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "paris", "is", "the", "capital", "of", "france", "where", "what", "berlin", "germany", "."]


def _word_tokenizer(path):
    tokenizers = pytest.importorskip("tokenizers")
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel({w: i for i, w in enumerate(VOCAB)}, unk_token="[UNK]"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    tok.post_processor = tokenizers.processors.TemplateProcessing(single="[CLS] $A [SEP]", pair="[CLS] $A [SEP] $B:1 [SEP]:1",
                                                                  special_tokens=[("[CLS]", 2), ("[SEP]", 3)])
    tok.add_special_tokens(["[MASK]"])                 # kept whole by the pre-tokenizer, as in real vocabularies
    tok.save(str(path))


def _tiny_repo(dst, hf_cls, arch, **extra):
    hc = transformers.BertConfig(vocab_size=len(VOCAB), hidden_size=32, num_hidden_layers=1, num_attention_heads=4, intermediate_size=64,
                                 max_position_embeddings=32, architectures=[arch], **extra)
    torch.manual_seed(0)
    model = hf_cls(hc).eval()
    dst.mkdir(parents=True, exist_ok=True)
    (dst / "config.json").write_text(hc.to_json_string())
    (dst / "model.safetensors").write_bytes(hf_state_bytes(model))
    _word_tokenizer(dst / "tokenizer.json")
    return model


def test_family_and_auto_classes_load_with_from_pretrained(tmp_path):
    from flodl_b200.hf.hub import HubExportHead
    from flodl_b200.hf.tokenizer import HfTokenizer
    repo = tmp_path / "tiny-bert"
    ref = _tiny_repo(repo, transformers.BertModel, "BertModel")
    ids = torch.tensor([[2, 5, 6, 7, 8, 3]])
    want = ref(ids).last_hidden_state
    g = bert.BertModel.from_pretrained(str(repo))                       # keeps the pooler the weights carry
    enc = HfTokenizer.from_pretrained(str(repo)).encode(["paris is the capital"])
    assert enc.input_ids.tolist() == ids.tolist()
    g.set_training(False)
    with torch.no_grad():
        out = g.forward_multi(bert.BertConfig.encoder_inputs(enc))
    assert out.t.shape == (1, 32)                                        # pooled output
    g2 = hf.AutoModel.from_pretrained(str(repo))                         # uniform [B, S, H] output
    g2.set_training(False)
    with torch.no_grad():
        torch.testing.assert_close(g2.forward_multi(bert.BertConfig.encoder_inputs(enc)).t, want, atol=1e-4, rtol=1e-4)
    assert json.loads(g2.source_config())["architectures"] == ["BertModel"]
    assert hf.AutoConfig.from_pretrained(str(repo)).model_type() == "bert"
    assert hf.AutoModel.from_pretrained_for_export(str(repo)).structural_hash() == g.structural_hash()
    g3 = hf.AutoModel.from_pretrained_for_export_with_head(str(repo), HubExportHead.Base)
    assert g3.structural_hash() == g.structural_hash()
    with pytest.raises(Exception, match="model_type"):
        roberta.RobertaModel.from_pretrained(str(repo))
    with pytest.raises(Exception):
        bert.BertModel.from_pretrained(str(tmp_path / "nope"))


def test_sequence_classification_predicts_from_text(tmp_path):
    repo = tmp_path / "cls"
    ref = _tiny_repo(repo, transformers.BertForSequenceClassification, "BertForSequenceClassification", num_labels=3,
                     id2label={0: "neg", 1: "neu", 2: "pos"}, label2id={"neg": 0, "neu": 1, "pos": 2})
    for head in (bert.BertForSequenceClassification.from_pretrained(str(repo)), hf.AutoModelForSequenceClassification.from_pretrained(str(repo))):
        assert head.labels() == ["neg", "neu", "pos"] and head.tokenizer is not None
        got = head.predict(["paris is the capital of france", "berlin"])
        assert len(got) == 2 and [k for k, _ in sorted(got[0])] == ["neg", "neu", "pos"]
        ids = head.tokenizer.encode(["paris is the capital of france"])
        want = torch.softmax(ref(ids.input_ids).logits, -1)[0]
        assert abs(dict(got[0])["pos"] - float(want[2])) < 1e-4 and got[0][0][1] >= got[0][1][1] >= got[0][2][1]
        assert head.classify(ids)[0][0][0] == got[0][0][0] and head.predict("berlin")[0][0][0] == got[1][0][0]
    bare = bert.BertForSequenceClassification.on_device(bert.BertConfig.from_json_str((repo / "config.json").read_text()), 3)
    with pytest.raises(Exception, match="needs a tokenizer"):
        bare.predict(["paris"])


def test_token_classification_returns_token_predictions(tmp_path):
    from flodl_b200.hf.task_heads import TokenPrediction
    repo = tmp_path / "tok"
    _tiny_repo(repo, transformers.BertForTokenClassification, "BertForTokenClassification", num_labels=3)
    head = hf.AutoModelForTokenClassification.from_pretrained(str(repo))
    rows = head.predict(["paris is the capital", "berlin"])
    assert len(rows) == 2 and len(rows[0]) == 6 and all(isinstance(p, TokenPrediction) for p in rows[0])
    assert [p.token for p in rows[0]] == ["[CLS]", "paris", "is", "the", "capital", "[SEP]"]
    assert [p.attends for p in rows[1]] == [True, True, True, False, False, False] and rows[0][1].label in ("LABEL_0", "LABEL_1", "LABEL_2")
    assert 1 / 3 <= rows[0][1].score <= 1.0


def test_question_answering_extracts_a_context_span(tmp_path):
    from flodl_b200.hf.task_heads import Answer
    repo = tmp_path / "qa"
    ref = _tiny_repo(repo, transformers.BertForQuestionAnswering, "BertForQuestionAnswering")
    head = bert.BertForQuestionAnswering.from_pretrained(str(repo))
    a = head.answer("what is the capital of france", "paris is the capital of france .")
    assert isinstance(a, Answer) and a.end >= a.start >= 8            # inside the context: [CLS] + 6 question tokens + [SEP]
    enc = head.tokenizer.encode_pairs([("what is the capital of france", "paris is the capital of france .")])
    assert enc.sequence_ids[0].tolist()[:9] == [-1, 0, 0, 0, 0, 0, 0, -1, 1]
    with torch.no_grad():
        o = ref(enc.input_ids, token_type_ids=enc.token_type_ids)
    ps, pe = torch.softmax(o.start_logits, 1)[0], torch.softmax(o.end_logits, 1)[0]
    ctx = [i for i, s in enumerate(enc.sequence_ids[0].tolist()) if s == 1]
    best = max(((i, j) for i in ctx for j in ctx if j >= i), key=lambda ij: float(ps[ij[0]] + pe[ij[1]]))
    assert (a.start, a.end) == best and abs(a.score - float(ps[best[0]] + pe[best[1]])) < 1e-4
    assert a.text == head.tokenizer.decode(enc.input_ids[0, a.start:a.end + 1].tolist())
    two = head.answer_batch([("where is paris", "paris is the capital of france"), ("what", "berlin germany")])
    assert len(two) == 2 and head.extract(enc)[0] == a
    single = head.tokenizer.encode(["paris"])
    with pytest.raises(Exception, match="no context tokens"):
        head.extract(single)


def test_fill_mask_from_text(tmp_path):
    repo = tmp_path / "mlm"
    ref = _tiny_repo(repo, transformers.BertForMaskedLM, "BertForMaskedLM")
    head = hf.AutoModelForMaskedLM.from_pretrained(str(repo))
    out = head.fill_mask("paris is the [MASK] of [MASK]", 3)
    assert len(out) == 2 and len(out[0]) == 3 and out[0][0][1] >= out[0][1][1] >= out[0][2][1] and out[0][0][0] in VOCAB
    enc = head.tokenizer.encode(["paris is the [MASK] of [MASK]"])
    with torch.no_grad():
        want = torch.softmax(ref(enc.input_ids).logits, -1)[0, 4]
    assert out[0][0][0] == VOCAB[int(want.argmax())] and abs(out[0][0][1] - float(want.max())) < 1e-4
    with pytest.raises(Exception, match="no \\[MASK\\]"):
        head.fill_mask("paris is", 2)
    with pytest.raises(Exception, match="top_k"):
        head.fill_mask("paris [MASK]", 0)
    pairs = head.fill_mask([enc.input_ids, enc.position_ids, enc.token_type_ids, bert.build_extended_attention_mask(enc.attention_mask)], [(0, 4)], 2)
    assert pairs[0][0][0] == int(want.argmax())
    g = hf.AutoModel.from_pretrained_for_export(str(repo))
    assert g.structural_hash() == head.graph().structural_hash()


def test_generic_heads_dispatch_on_the_config_family_and_small_names():
    from flodl_b200.hf.task_heads import ClassificationHead, MaskedLmHead, QaHead, TaggingHead
    cfg = distilbert.DistilBertConfig(vocab_size=30, dim=16, hidden_dim=32, n_layers=1, n_heads=2, max_position_embeddings=8)
    assert type(ClassificationHead.on_device(cfg, 2, None)).__name__ == "DistilBertForSequenceClassification"
    assert type(TaggingHead.on_device(cfg, 2, None)).__name__ == "DistilBertForTokenClassification"
    assert type(QaHead.on_device(cfg, None)).__name__ == "DistilBertForQuestionAnswering"
    assert type(MaskedLmHead.on_device(cfg, None)).__name__ == "DistilBertForMaskedLM"
    with pytest.raises(Exception, match="not a known family"):
        QaHead.on_device(object())
    assert HfPath.new("encoder").sub("layer").sub(3).path == "encoder.layer.3"


def test_deberta_stage_modules_match_the_fused_layer():
    from flodl_b200.autograd import Variable
    c = deberta_v2.DebertaV2LayerConfig(hidden_size=16, num_attention_heads=2, intermediate_size=32, hidden_dropout_prob=0.0,
                                        attention_probs_dropout_prob=0.0, layer_norm_eps=1e-7, position_buckets=8, max_relative_positions=16)
    so, it, out = (deberta_v2.DebertaV2SelfOutput.on_device(c), deberta_v2.DebertaV2Intermediate.on_device(c), deberta_v2.DebertaV2Output.on_device(c))
    x, r = Variable.wrap(torch.randn(2, 5, 16)), Variable.wrap(torch.randn(2, 5, 16))
    want = torch.nn.functional.layer_norm(torch.nn.functional.linear(x.t, so.dense.weight.t, so.dense.bias.t) + r.t, [16],
                                          so.layer_norm.weight.t, so.layer_norm.bias.t, 1e-7)
    torch.testing.assert_close(so.forward_pair(x, r).t, want, atol=1e-5, rtol=1e-5)
    up = it.forward(x)
    torch.testing.assert_close(up.t, torch.nn.functional.gelu(torch.nn.functional.linear(x.t, it.dense.weight.t, it.dense.bias.t)), atol=1e-5, rtol=1e-5)
    assert out.forward_pair(up, x).t.shape == (2, 5, 16)
    assert [p.name for p in so.parameters()] == ["dense.weight", "dense.bias", "LayerNorm.weight", "LayerNorm.bias"]
    assert [p.name for p in it.parameters()] == ["dense.weight", "dense.bias"] and out.dense.weight.t.shape == (16, 32)


# ---- export tool, export verification, stress parity ---------------------------------------------------------------
def test_deberta_log_buckets_match_transformers_inside_and_beyond_the_relative_range():
    from transformers.models.deberta_v2.modeling_deberta_v2 import make_log_bucket_position as theirs
    for bucket, maxp, seq in ((4, 8, 12), (8, 16, 40), (32, 64, 64), (256, 512, 512), (256, 512, 700)):
        ids = torch.arange(seq)
        rel = ids[:, None] - ids[None, :]
        mine = deberta_v2.make_log_bucket_position(rel, bucket, maxp)
        assert torch.equal(mine, theirs(rel, bucket, maxp).long()), (bucket, maxp, seq)


@pytest.mark.parametrize("family", ["bert", "albert", "deberta-v2"])
def test_parity_holds_with_weights_of_trained_size_and_long_sequences(family):
    """Initialiser-sized weights (std 0.02) keep every attention score near zero and can hide a wrong term; std 0.3 cannot."""
    from flodl_b200.hf import parity
    for head in ("base", "mlm"):
        worst, note = parity.compare(family, head, stress=True, seq_len=20)
        assert note is None and worst < 1e-3, (family, head, worst, note)


def test_deberta_config_emits_and_checks_legacy():
    cfg = deberta_v2.DebertaV2Config(vocab_size=40, hidden_size=16, num_hidden_layers=1, num_attention_heads=2, intermediate_size=32,
                                     max_position_embeddings=16, position_buckets=4, max_relative_positions=8)
    emitted = json.loads(cfg.to_json_str())
    assert emitted["legacy"] is False
    assert deberta_v2.DebertaV2Config.from_json_str(cfg.to_json_str()).hidden_size == 16
    emitted["legacy"] = True
    assert deberta_v2.DebertaV2Config.from_json_str(json.dumps(emitted)).hidden_size == 16     # irrelevant for the encoder: ignored
    emitted["architectures"] = ["DebertaV2ForMaskedLM"]
    with pytest.raises(Exception, match="legacy = true is not supported"):
        deberta_v2.DebertaV2Config.from_json_str(json.dumps(emitted))


def test_export_tool_hub_and_checkpoint_modes_and_verify_export(tmp_path, capsys):
    from flodl_b200.hf import export_tool, verify_export
    repo = tmp_path / "src"
    _tiny_repo(repo, transformers.BertForSequenceClassification, "BertForSequenceClassification", num_labels=3)
    out = str(tmp_path / "exp")
    assert export_tool.main(["--hub", str(repo), "--out", out]) == 0
    cfg = json.loads(open(os.path.join(out, "config.json")).read())
    assert cfg["flodl_source_repo"] == str(repo) and cfg["architectures"] == ["BertForSequenceClassification"]
    rep = verify_export.verify(out)                                   # the stamped source is found and compared bit for bit
    assert rep["ok"] and rep["loadable"] and rep["source_parity"] and rep["max_abs_diff_vs_source"] == 0.0 and rep["hub_source"] == str(repo)
    assert rep["auto_class"] == "AutoModelForSequenceClassification" and rep["max_abs_diff_vs_transformers"] < 1e-4
    base = str(tmp_path / "exp_base")
    assert export_tool.main(["--hub", str(repo), "--out", base, "--head", "base"]) == 0     # a head checkpoint re-exported as an encoder
    assert json.loads(open(os.path.join(base, "config.json")).read())["architectures"] == ["BertModel"]
    assert verify_export.main([base, "--no-hub-source"]) == 0
    capsys.readouterr()
    # checkpoint mode: a graph saved as .fdl with its config sidecar
    head = bert.BertForTokenClassification.on_device(bert.BertConfig.from_json_str((repo / "config.json").read_text()), 3)
    ck = str(tmp_path / "m.fdl")
    head.graph().save_checkpoint(ck)
    out2 = str(tmp_path / "exp2")
    assert export_tool.main(["--checkpoint", ck, "--out", out2]) == 0
    assert verify_export.main([out2]) == 2 and "no upstream to compare with" in capsys.readouterr().err
    assert verify_export.main([out2, "--no-hub-source"]) == 0
    assert json.loads(capsys.readouterr().out)["architecture"] == "BertForTokenClassification"
    assert export_tool.main(["--out", out2]) == 2 and "exactly one of" in capsys.readouterr().err
    assert export_tool.main(["--checkpoint", ck, "--head", "qa", "--out", out2]) == 2
    assert verify_export.auto_class_for("XLMRobertaForQuestionAnswering") == ("AutoModelForQuestionAnswering", "qa")
    assert verify_export.auto_class_for("AlbertModel") == ("AutoModel", "base")
    with pytest.raises(Exception, match="unsupported architecture"):
        verify_export.auto_class_for("BertForPreTraining")


def test_verify_export_flags_a_damaged_export(tmp_path):
    from flodl_b200.hf import export_tool, verify_export
    repo = tmp_path / "src"
    _tiny_repo(repo, transformers.BertModel, "BertModel")
    out = str(tmp_path / "exp")
    export_tool.export_from_hub(str(repo), out)
    tensors = st.read_safetensors(open(os.path.join(out, "model.safetensors"), "rb").read())
    key = next(k for k in tensors if k.endswith("attention.self.query.weight"))
    tensors["encoder.layer.0.attention.self.queri.weight"] = tensors.pop(key)          # a renamed key: one missing, one unexpected
    open(os.path.join(out, "model.safetensors"), "wb").write(st.write_safetensors(tensors))
    rep_keys = verify_export._load_with_transformers(transformers, "AutoModel", out)
    assert any("query.weight" in k for k in rep_keys[1]) and any("queri" in k for k in rep_keys[2])


def test_export_verification_matrix_cells(tmp_path):
    from flodl_b200.hf import verify_export
    res = verify_export.verify_matrix(["distilbert", "deberta-v2"], ["base", "qa", "mlm"], str(tmp_path / "stage"), keep=True)
    assert all(not isinstance(r, str) and r["ok"] for r in res.values()), res
    assert os.path.isfile(tmp_path / "stage" / "deberta-v2-mlm" / "model.safetensors")
    grid = verify_export.render_matrix(res, ["distilbert", "deberta-v2"], ["base", "qa", "mlm"])
    assert grid.count("PASS") == 6 and "FAIL" not in grid


# ---- runnable demos, on local tiny repos --------------------------------------------------------------------------------
def test_examples_list_and_run_on_local_repos(tmp_path, capsys):
    from flodl_b200.hf import examples
    assert examples.main([]) == 0
    listing = capsys.readouterr().out
    for name in ("auto-classify", "bert-embed", "bert-classify", "bert-ner", "bert-qa", "roberta-embed", "roberta-qa", "distilbert-classify",
                 "distilbert-ner", "distilbert-finetune"):
        assert name in listing
    assert len(examples.EXAMPLES) == 14
    assert examples.main(["nope"]) == 2
    lines = []
    base = tmp_path / "base"
    _tiny_repo(base, transformers.BertModel, "BertModel")
    emb = examples.embed(str(base), ["paris is the capital", "berlin", "paris is the capital"], lines.append)
    assert emb.shape == (3, 32) and torch.allclose(emb[0], emb[2], atol=1e-5) and abs(float(emb[0] @ emb[0]) - 1.0) < 1e-5
    cls = tmp_path / "cls"
    _tiny_repo(cls, transformers.BertForSequenceClassification, "BertForSequenceClassification", num_labels=2, id2label={0: "neg", 1: "pos"},
               label2id={"neg": 0, "pos": 1})
    assert examples.main(["auto-classify", "--repo", str(cls), "paris is the capital", "berlin"]) == 0
    out = capsys.readouterr().out
    assert out.count("\n") == 2 and ("neg" in out or "pos" in out)
    tok = tmp_path / "tok"
    _tiny_repo(tok, transformers.BertForTokenClassification, "BertForTokenClassification", num_labels=3)
    assert len(examples.ner(str(tok), ["paris is the capital of france"], lines.append)[0]) == 8
    qa_repo = tmp_path / "qa"
    _tiny_repo(qa_repo, transformers.BertForQuestionAnswering, "BertForQuestionAnswering")
    assert examples.main(["bert-qa", "--repo", str(qa_repo), "where is paris", "paris is the capital of france"]) == 0
    assert "Q: where is paris" in capsys.readouterr().out
    assert examples.main(["bert-qa", "--repo", str(tmp_path / "missing")]) == 1


def test_finetune_example_lowers_the_loss_and_exports(tmp_path):
    from flodl_b200.hf import examples, verify_export
    cls = tmp_path / "cls"
    _tiny_repo(cls, transformers.BertForSequenceClassification, "BertForSequenceClassification", num_labels=2, id2label={0: "neg", 1: "pos"},
               label2id={"neg": 0, "pos": 1}, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    lines = []
    out_dir = str(tmp_path / "tuned")
    curve, preds = examples.finetune(str(cls), ["paris is the capital", "berlin germany", "france", "where what"], [1, 0, 1, 0], steps=30, lr=5e-3,
                                     out=lines.append, export_dir=out_dir)
    assert curve[-1] < 0.5 * curve[0] and preds == ["pos", "neg", "pos", "neg"]
    rep = verify_export.verify(out_dir, no_hub_source=True)
    assert rep["ok"] and rep["architecture"] == "BertForSequenceClassification"


def test_safetensors_reader_refuses_damaged_files_cleanly():
    """Random damage to a valid file, and hand-made hostile headers: the reader loads or raises TensorError, nothing else."""
    import json as _json, struct as _struct
    pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st
    from flodl_b200.hf.safetensors_io import read_safetensors, write_safetensors
    from flodl_b200.tensor import TensorError
    good = write_safetensors({"a.weight": torch.arange(12.0).view(3, 4), "a.bias": torch.zeros(4, dtype=torch.bfloat16), "s": torch.tensor(2.0)})
    assert set(read_safetensors(good)) == {"a.weight", "a.bias", "s"}

    def with_header(h, payload=b"\\0" * 64):
        raw = _json.dumps(h).encode()
        return _struct.pack("<Q", len(raw)) + raw + payload
    for hostile in ([1, 2], {"w": 3}, {"w": {"dtype": "F32", "shape": [2], "data_offsets": [-8, 0]}}, {"w": {"dtype": "F32", "shape": [-2, -4], "data_offsets": [0, 32]}},
                    {"w": {"dtype": "F32", "shape": [2]}}, {"w": {"dtype": 7, "shape": [2], "data_offsets": [0, 8]}}, {"w": {"dtype": "F32", "shape": [1 << 62, 4], "data_offsets": [0, 8]}},
                    {"w": {"dtype": "F32", "shape": "2", "data_offsets": [0, 8]}}, {"w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 1 << 40]}}):
        with pytest.raises(TensorError):
            read_safetensors(with_header(hostile))

    @settings(max_examples=300, deadline=None, derandomize=True, database=None)
    @given(st.lists(st.tuples(st.sampled_from(["flip", "cut", "noise"]), st.integers(0, len(good) - 1), st.binary(min_size=1, max_size=16)), min_size=1, max_size=3))
    def run(edits):
        data = bytearray(good)
        for kind, at, arg in edits:
            if not data:
                break
            at = min(at, len(data) - 1)
            if kind == "flip":
                data[at] ^= arg[0] or 1
            elif kind == "cut":
                del data[at:]
            else:
                data[at:at + len(arg)] = arg
        try:
            out = read_safetensors(bytes(data))
        except TensorError:
            return
        assert all(t.numel() * t.element_size() <= len(data) for t in out.values())
    run()
