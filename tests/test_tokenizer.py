"""The optional text path: a tokenizer.json made here with the `tokenizers` package (a word-level
vocabulary of 300 words, a post-processor that puts BOS first), read back by the engine's wrapper.
Encoding prepends BOS, decoding skips special tokens (crates/engine/src/tokenizer.rs:25-38)."""
import json
import os

import pytest

tokenizers = pytest.importorskip("tokenizers")

BOS, EOS, UNK = "<|begin_of_text|>", "<|end_of_text|>", "<unk>"


def make_tokenizer_json(folder) -> dict:
    """Write <folder>/tokenizer.json; returns the vocabulary {word: id}."""
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    from tokenizers.processors import TemplateProcessing
    words = [f"w{i}" for i in range(297)]
    vocab = {BOS: 0, EOS: 1, UNK: 2}
    vocab.update({w: 3 + i for i, w in enumerate(words)})
    tok = Tokenizer(WordLevel(vocab, unk_token=UNK))
    tok.pre_tokenizer = Whitespace()
    tok.add_special_tokens([BOS, EOS])
    tok.post_processor = TemplateProcessing(single=f"{BOS} $A", special_tokens=[(BOS, 0)])
    from tokenizers.decoders import WordPiece
    tok.decoder = WordPiece(prefix="##", cleanup=False)         # joins words with spaces
    os.makedirs(folder, exist_ok=True)
    tok.save(os.path.join(str(folder), "tokenizer.json"))
    return vocab


def test_encode_puts_bos_first_and_decode_skips_specials(tmp_path):
    from vllm_oxide_b200.engine.tokenizer import TextTokenizer
    vocab = make_tokenizer_json(tmp_path)
    assert len(vocab) == 300
    t = TextTokenizer.load(str(tmp_path))
    ids = t.encode("w5 w17 w296 nosuchword")
    assert ids == [0, vocab["w5"], vocab["w17"], vocab["w296"], vocab[UNK]]            # BOS first
    assert t.decode(ids[:4]) == "w5 w17 w296"                                             # BOS skipped
    assert t.decode([vocab["w1"], vocab["w2"], 1]) == "w1 w2"                             # EOS skipped
    assert t.encode("") == [0]


def test_folder_without_tokenizer_and_broken_file(tmp_path):
    from vllm_oxide_b200.engine.tokenizer import TextTokenizer, TokenizerError
    assert TextTokenizer.load(str(tmp_path)) is None
    (tmp_path / "tokenizer.json").write_text("{not a tokenizer")
    with pytest.raises(TokenizerError, match="tokenizer.json"):
        TextTokenizer.load(str(tmp_path))
