"""Byte-level BPE tokenizer of a GGUF checkpoint (host code): the reference's own fixture
(models/kalosm-llama/src/gguf_tokenizer.rs:595-860: a 256-byte vocabulary plus <s> / </s>, its
sample strings, encode and decode with and without special tokens), pinned a second time against
the `tokenizers` package (the library the reference's tests compare with), and the chat template."""
import numpy as np
import pytest

from kalosm_b200 import gguf
from kalosm_b200.tokenizer import GgufTokenizer, TokenizerError, bytes_to_unicode

SAMPLES = ["Hello world", "  leading spaces and\ttabs\n\nnewlines", "naïve café — 你好, мир! 12345 67",
           "it's we're I'll DON'T", "code::{ let x = 12345; }\r\nnext", "<s>Hello</s>   tail",
           "tabs\t\tword and spaces   word"]


def byte_vocab():
    b2u = bytes_to_unicode()
    tokens = [b2u[b] for b in range(256)] + ["<s>", "</s>"]
    types = [1] * 256 + [3, 3]
    return tokens, types


@pytest.mark.parametrize("pre", ["llama-bpe", "qwen2", "gpt-2", "something-unknown"])
def test_byte_vocabulary_fixture(pre):
    tokens, types = byte_vocab()
    tok = GgufTokenizer(tokens, (), types, bos_token_id=256, eos_token_id=257, pre=pre)
    for text in SAMPLES:
        for add in (False, True):
            ids = tok.encode(text, add_special_tokens=add)
            # without merges every byte is its own token; <s> and </s> are matched as wholes
            want, rest = ([256] if add else []), text
            while rest:
                if rest.startswith("<s>"):
                    want.append(256); rest = rest[3:]
                elif rest.startswith("</s>"):
                    want.append(257); rest = rest[4:]
                else:
                    want += list(rest[0].encode("utf-8")); rest = rest[1:]
            assert ids == want, (pre, text)
            assert tok.decode(ids) == ("<s>" if add else "") + text
            assert tok.decode(ids, skip_special_tokens=True) == text.replace("<s>", "").replace("</s>", "")
    assert tok.is_special_token(256) and not tok.is_special_token(65)
    assert tok.decode([0xE4, 0xBD]) == "�"  # a cut UTF-8 sequence is replaced, not an error


def _hf_tokenizer(tokens, merges, pattern):
    tk = pytest.importorskip("tokenizers")
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers
    vocab = {t: i for i, t in enumerate(tokens)}
    t = Tokenizer(models.BPE(vocab=vocab, merges=[tuple(m.split(" ")) for m in merges], ignore_merges=False))
    t.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pattern), behavior="isolated"),
                                               pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    t.decoder = decoders.ByteLevel()
    return t


def test_merges_against_the_tokenizers_package():
    # a vocabulary with learned merges: same ids as the `tokenizers` BPE with the same split pattern
    from kalosm_b200.tokenizer import PRE_TOKENIZER_PATTERNS
    b2u = bytes_to_unicode()
    base = [b2u[b] for b in range(256)]
    sp = b2u[ord(" ")]
    merges = ["h e", "l l", "he ll", "hell o", f"{sp} w", "o r", f"{sp}w or", "l d", f"{sp}wor ld", "1 2", "12 3",
              f"{sp} hello", "t h", "th e", f"{sp} the", "i n", "in g"]
    tokens = list(base)
    for m in merges:
        a, b = m.split(" ")
        if a + b not in tokens:
            tokens.append(a + b)
    ours = GgufTokenizer(tokens, merges, None, pre="qwen2", add_bos=False)
    hf = _hf_tokenizer(tokens, merges, PRE_TOKENIZER_PATTERNS["qwen2"][0])
    for text in SAMPLES + ["hello world", "the hello world thing 123 1234", "hellohello  world\nworld"]:
        text = text.replace("<s>", "").replace("</s>", "")
        assert ours.encode(text, add_special_tokens=False) == hf.encode(text, add_special_tokens=False).ids, text
        assert ours.decode(ours.encode(text, add_special_tokens=False)) == text
    # ignore_merges (llama3 family, gguf_tokenizer.rs:458-463): a piece that is a vocabulary entry
    # is emitted whole even when the merge list could not build it
    llama = GgufTokenizer(tokens + [f"{sp}thing"], merges, None, pre="llama-bpe", add_bos=False)
    assert llama.encode(" thing", add_special_tokens=False) == [len(tokens)]
    plain = GgufTokenizer(tokens + [f"{sp}thing"], merges, None, pre="qwen2", add_bos=False)
    assert len(plain.encode(" thing", add_special_tokens=False)) > 1


def test_llama3_split_pattern():
    tokens, types = byte_vocab()
    tok = GgufTokenizer(tokens, (), types, pre="llama-bpe")
    assert tok._split("Hello world's 1234567 !!\n\n  x") == ["Hello", " world", "'s", " ", "123", "456", "7", " !!\n\n", " ", " x"]


def test_from_gguf_and_chat_template(tmp_path):
    tokens, types = byte_vocab()
    template = ("{{ bos_token }}{% for m in messages %}<|{{ m['role'] }}|>\n{{ m['content'] }}{{ eos_token }}\n"
                "{% endfor %}{% if add_generation_prompt %}<|assistant|>\n{% endif %}")
    md = {"general.architecture": (gguf.STRING, "llama"), "tokenizer.ggml.model": (gguf.STRING, "gpt2"),
          "tokenizer.ggml.pre": (gguf.STRING, "llama-bpe"),
          "tokenizer.ggml.tokens": (gguf.ARRAY, (gguf.STRING, tokens)),
          "tokenizer.ggml.token_type": (gguf.ARRAY, (gguf.I32, types)),
          "tokenizer.ggml.merges": (gguf.ARRAY, (gguf.STRING, [])),
          "tokenizer.ggml.bos_token_id": (gguf.U32, 256), "tokenizer.ggml.eos_token_id": (gguf.U32, 257),
          "tokenizer.chat_template": (gguf.STRING, template)}
    path = tmp_path / "tok.gguf"
    gguf.write_gguf(path, md, [("v", (4,), 0, np.zeros(4, np.float32))])
    tok = GgufTokenizer.from_gguf(gguf.GgufFile(path))
    assert tok.encode("hi") == [256, ord("h"), ord("i")]
    text = tok.apply_chat_template([{"role": "user", "content": "hi"}])
    assert text == "<s><|user|>\nhi</s>\n<|assistant|>\n"
    ids = tok.encode(text, add_special_tokens=False)
    assert ids[0] == 256 and 257 in ids and tok.decode(ids) == text
    bare = GgufTokenizer(tokens, (), types)
    with pytest.raises(TokenizerError):
        bare.apply_chat_template([{"role": "user", "content": "x"}])
