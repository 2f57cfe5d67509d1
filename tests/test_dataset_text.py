"""Text transforms, vocabularies and vector tables."""
import numpy as np
import pytest

import mindspore_b200.dataset as ds
from mindspore_b200.dataset import text


def test_vocab_and_lookup(tmp_path):
    v = text.Vocab.from_list(["cat", "dog"], special_tokens=["<pad>", "<unk>"], special_first=True)
    assert v.vocab() == {"<pad>": 0, "<unk>": 1, "cat": 2, "dog": 3} and len(v) == 4
    assert v.tokens_to_ids(["dog", "emu"]) == [3, -1] and v.ids_to_tokens([2, 0]) == ["cat", "<pad>"]
    look = text.Lookup(v, unknown_token="<unk>")
    assert look(np.array(["cat", "emu", "dog"])).tolist() == [2, 1, 3]
    with pytest.raises(RuntimeError):
        text.Lookup(v)(np.array(["emu"]))
    with pytest.raises(ValueError):
        text.Vocab.from_list(["a", "a"])
    (tmp_path / "v.txt").write_text("apple,1\nbanana,2\ncherry,3\n")
    vf = text.Vocab.from_file(str(tmp_path / "v.txt"), delimiter=",", vocab_size=2, special_tokens=["<unk>"],
                              special_first=False)
    assert vf.vocab() == {"apple": 0, "banana": 1, "<unk>": 2}
    data = ds.NumpySlicesDataset({"t": np.array([["b", "a"], ["b", "c"]], dtype=object)}, shuffle=False)
    vd = text.Vocab.from_dataset(data, "t", freq_range=(1, None), top_k=2)
    assert vd.vocab() == {"b": 0, "a": 1}
    assert text.Vocab.from_dict({"x": 1, "y": 0}).ids_to_tokens(1) == "x"


def test_tokenizers():
    t = np.array("Welcome to  Beijing!")
    assert text.WhitespaceTokenizer()(t).tolist() == ["Welcome", "to", "Beijing!"]
    toks, start, limit = text.WhitespaceTokenizer(with_offsets=True)(t)
    assert start.tolist() == [0, 8, 12] and limit.tolist() == [7, 10, 20]
    assert text.UnicodeCharTokenizer()(np.array("ab c")).tolist() == ["a", "b", " ", "c"]
    assert text.UnicodeScriptTokenizer()(np.array("Hi, 北京 42")).tolist() == ["Hi", ",", "北京", "42"]
    assert text.RegexTokenizer(r"\s+|,", ",")(np.array("a, b")).tolist() == ["a", ",", "b"]
    assert str(text.RegexReplace(r"\d+", "#")(np.array("a1b22"))) == "a#b#"
    assert text.CaseFold()(np.array(["ÀB", "ß"])).tolist() == ["àb", "ss"]
    assert str(text.NormalizeUTF8(text.NormalizeForm.NFKC)(np.array("ｆｉ"))) == "fi"
    basic = text.BasicTokenizer(lower_case=True)
    assert basic(np.array("Héllo, [UNK] 世界!")).tolist() == ["hello", ",", "[UNK]", "世", "界", "!"]
    vocab = text.Vocab.from_list(["un", "##want", "##ed", "run", "##ning", ",", "[UNK]"])
    wp = text.WordpieceTokenizer(vocab)
    assert wp(np.array(["unwanted", "running", "xyz"])).tolist() == ["un", "##want", "##ed", "run", "##ning", "[UNK]"]
    bert = text.BertTokenizer(vocab, lower_case=True)
    assert bert(np.array("Unwanted, running")).tolist() == ["un", "##want", "##ed", ",", "run", "##ning"]
    pieces, s, l = text.BertTokenizer(vocab, lower_case=True, with_offsets=True)(np.array("unwanted running"))
    assert s.tolist() == [0, 2, 6, 9, 12] and l.tolist() == [2, 6, 8, 12, 16]
    assert text.PythonTokenizer(lambda s: s.split("-"))(np.array("a-b")).tolist() == ["a", "b"]
    with pytest.raises(TypeError):
        text.PythonTokenizer(3)
    with pytest.raises(RuntimeError):
        text.WhitespaceTokenizer()(np.array(["a", "b"]))
    assert str(text.FilterWikipediaXML()(np.array("<p>Hello [[World|W]] 2</p>"))) == "hello w two"


def test_sentencepiece(tmp_path):
    corpus = tmp_path / "c.txt"
    corpus.write_text("\n".join(["the quick brown fox jumps over the lazy dog"] * 50 + ["pack my box with jugs"] * 50))
    vocab = text.SentencePieceVocab.from_file([str(corpus)], 30, 1.0, text.SentencePieceModel.UNIGRAM, {})
    tok = text.SentencePieceTokenizer(vocab, text.SPieceTokenizerOutType.STRING)
    pieces = tok(np.array("the quick fox")).tolist()
    assert "".join(pieces).replace("▁", " ").strip() == "the quick fox"
    ids = text.SentencePieceTokenizer(vocab, text.SPieceTokenizerOutType.INT)(np.array("the quick fox"))
    assert ids.dtype == np.int32 and len(ids) == len(pieces)
    text.SentencePieceVocab.save_model(vocab, str(tmp_path), "m.model")
    again = text.SentencePieceTokenizer(str(tmp_path / "m.model"), text.SPieceTokenizerOutType.STRING)
    assert again(np.array("the quick fox")).tolist() == pieces


def test_sequence_helpers_and_vectors(tmp_path):
    toks = np.array(["a", "b", "c"])
    assert text.Ngram(2)(toks).tolist() == ["a b", "b c"]
    assert text.Ngram([1, 2], ("_", 1), ("_", 1), "-")(toks).tolist() == ["a", "b", "c", "_-a", "a-b", "b-c", "c-_"]
    assert text.SlidingWindow(2)(np.array([1, 2, 3, 4])).tolist() == [[1, 2], [2, 3], [3, 4]]
    assert text.Truncate(2)(toks).tolist() == ["a", "b"]
    a, b = text.TruncateSequencePair(4)(np.array([1, 2, 3]), np.array([4, 5, 6]))
    assert len(a) + len(b) == 4 and a.tolist() == [1, 2] and b.tolist() == [4, 5]
    assert text.AddToken("<s>")(toks).tolist() == ["<s>", "a", "b", "c"]
    assert text.AddToken("</s>", begin=False)(toks).tolist() == ["a", "b", "c", "</s>"]
    assert text.ToNumber(np.int32)(np.array(["1", "-2"])).tolist() == [1, -2]
    assert text.ToNumber(np.float32)(np.array("2.5")).item() == 2.5
    with pytest.raises(RuntimeError):
        text.ToNumber(np.int8)(np.array(["300"]))
    (tmp_path / "vec.txt").write_text("2 3\nok 1 2 3\nhi 4 5 6\n")
    vec = text.Vectors.from_file(str(tmp_path / "vec.txt"))
    assert vec.dim == 3
    tv = text.ToVectors(vec, unk_init=[9, 9, 9], lower_case_backup=True)
    assert tv(np.array(["OK", "no"])).tolist() == [[1, 2, 3], [9, 9, 9]]
    (tmp_path / "ng.txt").write_text("2gram-ab 1 1\n2gram-b#END# 3 3\n")
    cg = text.CharNGram.from_file(str(tmp_path / "ng.txt"))
    assert text.ToVectors(cg)(np.array("ab")).tolist() == [2, 2]
    assert text.to_str(text.to_bytes(np.array(["é"]))).tolist() == ["é"]
    data = ds.NumpySlicesDataset({"t": np.array(["a b", "c d e"], dtype=object)}, shuffle=False)
    data = data.map(text.WhitespaceTokenizer(), input_columns=["t"])
    assert [r["t"].tolist() for r in data.create_dict_iterator(output_numpy=True, num_epochs=1)] == [["a", "b"], ["c", "d", "e"]]
