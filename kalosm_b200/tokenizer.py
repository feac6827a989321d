"""Byte-level BPE tokenizer and chat template read from a GGUF checkpoint: text in, token ids out
(and back), the step in front of the embedding lookup.

Follows the reference's GGUF tokenizer (models/kalosm-llama/src/gguf_tokenizer.rs): the vocabulary
`tokenizer.ggml.tokens` in the GPT-2 byte-to-unicode alphabet, `tokenizer.ggml.merges` as ranked
pairs, special tokens = every token whose `tokenizer.ggml.token_type` is not 1 (normal) plus BOS and
EOS (:284-300), matched longest-first at every text offset before anything else (:437-443); normal
text is cut by the pre-tokenizer's regular expressions (`tokenizer.ggml.pre`, :44-125 and :454-590)
and every piece is merged by rank (kalosm-tokenizer's FastBpe); with `ignore_merges` (the llama3
and tekken families) a piece that is a vocabulary entry as a whole becomes that single token.
Decoding concatenates the tokens' bytes and replaces invalid UTF-8 (:387-398). The chat template
(models/kalosm-llama/src/chat_template.rs) is the checkpoint's Jinja template rendered with
`messages`, `bos_token`, `eos_token` and `add_generation_prompt`.

Host code only; nothing here touches the GPU.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import regex

# Split patterns per pre-tokenizer family (gguf_tokenizer.rs:44-125). Families not listed fall back
# to the default (GPT-2) pattern, as the reference's `Default` variant does.
_GPT2 = r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)"
PRE_TOKENIZER_PATTERNS: Dict[str, Tuple[str, ...]] = {
    "llama3": (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+",),
    "qwen2": (r"(?:'[sS]|'[tT]|'[rR][eE]|'[vV][eE]|'[mM]|'[lL][lL]|'[dD])|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+",),
    "gpt2": (_GPT2,),
    "default": (_GPT2,),
}
# `tokenizer.ggml.pre` labels -> (family, ignore_merges, add_bos) (gguf_tokenizer.rs:454-590)
PRE_TOKENIZER_LABELS = {
    "llama3": ("llama3", True, True), "llama-v3": ("llama3", True, True), "llama-bpe": ("llama3", True, True),
    "falcon3": ("llama3", True, True), "qwen2": ("qwen2", False, True), "qwen3": ("qwen2", False, True),
    "gpt-2": ("gpt2", False, True), "phi-2": ("gpt2", False, True), "roberta-bpe": ("gpt2", False, True),
}


def bytes_to_unicode() -> Dict[int, str]:
    """The GPT-2 byte-level alphabet: printable bytes map to themselves, the rest to U+0100 upwards
    in byte order (restated in the reference's tests, gguf_tokenizer.rs:814-834)."""
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


_B2U = bytes_to_unicode()
_U2B = {c: b for b, c in _B2U.items()}


class TokenizerError(ValueError):
    pass


class GgufTokenizer:
    """Byte-level BPE over a GGUF vocabulary."""

    def __init__(self, tokens: Sequence[str], merges: Iterable[str] = (), token_types: Optional[Sequence[int]] = None,
                 bos_token_id: Optional[int] = None, eos_token_id: Optional[int] = None, pre: str = "default",
                 add_bos: Optional[bool] = None, chat_template: Optional[str] = None):
        self.tokens = list(tokens)
        self.vocab = {t: i for i, t in enumerate(self.tokens)}
        family, ignore_merges, default_add_bos = PRE_TOKENIZER_LABELS.get(pre, ("default", False, True))
        self.patterns = [regex.compile(p) for p in PRE_TOKENIZER_PATTERNS[family]]
        self.ignore_merges = ignore_merges
        self.add_bos = default_add_bos if add_bos is None else bool(add_bos)
        self.bos_token_id, self.eos_token_id = bos_token_id, eos_token_id
        self.chat_template = chat_template
        self.ranks: Dict[Tuple[str, str], int] = {}
        for rank, m in enumerate(merges):
            left, _, right = m.partition(" ")
            self.ranks.setdefault((left, right), rank)
        types = list(token_types) if token_types is not None else [1] * len(self.tokens)
        # special = not a normal token, or BOS / EOS (gguf_tokenizer.rs:284-296); matched longest first
        self.special = [False] * len(self.tokens)
        by_first: Dict[int, List[Tuple[bytes, int]]] = {}
        for i, t in enumerate(self.tokens):
            ty = types[i] if i < len(types) else 1
            if ty != 1 or i == bos_token_id or i == eos_token_id:
                self.special[i] = True
                raw = t.encode("utf-8")
                if raw:
                    by_first.setdefault(raw[0], []).append((raw, i))
        for bucket in by_first.values():
            bucket.sort(key=lambda e: -len(e[0]))
        self._special_by_first = by_first
        # bytes of every token for decoding: specials are their literal text, others the byte alphabet
        self._token_bytes: List[bytes] = []
        for i, t in enumerate(self.tokens):
            if self.special[i] or any(c not in _U2B for c in t):
                self._token_bytes.append(t.encode("utf-8"))
            else:
                self._token_bytes.append(bytes(_U2B[c] for c in t))

    # ---- construction from a checkpoint ----------------------------------------------------------
    @classmethod
    def from_gguf(cls, g) -> "GgufTokenizer":
        """`g`: a kalosm_b200.gguf.GgufFile. Keys as Model::from_var_source reads them
        (models/kalosm-llama/src/raw/mod.rs:332-372)."""
        md = g.metadata
        if "tokenizer.ggml.tokens" not in md:
            raise TokenizerError("the file has no tokenizer.ggml.tokens")
        model = md.get("tokenizer.ggml.model", "gpt2")
        if model != "gpt2":
            raise TokenizerError(f"tokenizer model {model!r} is not byte-level BPE")
        return cls(md["tokenizer.ggml.tokens"], md.get("tokenizer.ggml.merges", ()),
                   md.get("tokenizer.ggml.token_type"), md.get("tokenizer.ggml.bos_token_id"),
                   md.get("tokenizer.ggml.eos_token_id"), md.get("tokenizer.ggml.pre", "default"),
                   md.get("tokenizer.ggml.add_bos_token"), md.get("tokenizer.chat_template"))

    # ---- encoding --------------------------------------------------------------------------------
    def _split(self, text: str) -> List[str]:
        pieces = [text]
        for pat in self.patterns:  # every pattern isolates its matches; what lies between stays a piece
            nxt: List[str] = []
            for piece in pieces:
                pos = 0
                for m in pat.finditer(piece):
                    if m.end() == m.start():
                        continue
                    if m.start() > pos:
                        nxt.append(piece[pos:m.start()])
                    nxt.append(m.group())
                    pos = m.end()
                if pos < len(piece):
                    nxt.append(piece[pos:])
            pieces = nxt
        return pieces

    def _bpe(self, piece: str, out: List[int]) -> None:
        word = "".join(_B2U[b] for b in piece.encode("utf-8"))
        if self.ignore_merges and word in self.vocab:
            out.append(self.vocab[word])
            return
        syms = list(word)
        while len(syms) > 1:
            best, best_rank = -1, None
            for i in range(len(syms) - 1):
                r = self.ranks.get((syms[i], syms[i + 1]))
                if r is not None and (best_rank is None or r < best_rank):
                    best, best_rank = i, r
            if best < 0:
                break
            syms[best:best + 2] = [syms[best] + syms[best + 1]]
        for s in syms:
            if s not in self.vocab:
                raise TokenizerError(f"symbol {s!r} is not in the vocabulary")
            out.append(self.vocab[s])

    def _encode_normal(self, text: str, out: List[int]) -> None:
        if text:
            for piece in self._split(text):
                if piece:
                    self._bpe(piece, out)

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        out: List[int] = []
        if add_special_tokens and self.add_bos and self.bos_token_id is not None:
            out.append(self.bos_token_id)
        raw = text.encode("utf-8")
        offset = normal_start = 0
        while offset < len(raw):
            hit = None
            for tok, tid in self._special_by_first.get(raw[offset], ()):
                if raw.startswith(tok, offset):
                    hit = (len(tok), tid)
                    break
            if hit:
                self._encode_normal(raw[normal_start:offset].decode("utf-8"), out)
                out.append(hit[1])
                offset += hit[0]
                normal_start = offset
            else:
                offset += 1
                while offset < len(raw) and (raw[offset] & 0xC0) == 0x80:  # step over a whole character
                    offset += 1
        self._encode_normal(raw[normal_start:].decode("utf-8"), out)
        return out

    # ---- decoding --------------------------------------------------------------------------------
    def is_special_token(self, token: int) -> bool:
        return 0 <= token < len(self.special) and self.special[token]

    def decode(self, tokens: Iterable[int], skip_special_tokens: bool = False) -> str:
        data = bytearray()
        for t in tokens:
            t = int(t)
            if skip_special_tokens and self.is_special_token(t):
                continue
            if 0 <= t < len(self._token_bytes):
                data += self._token_bytes[t]
        return data.decode("utf-8", errors="replace")

    # ---- chat template ---------------------------------------------------------------------------
    def apply_chat_template(self, messages: Sequence[Dict[str, str]], add_generation_prompt: bool = True) -> str:
        """Renders the checkpoint's Jinja chat template (chat_template.rs:15-120: `messages`,
        `bos_token`, `eos_token`, `add_generation_prompt`, and `raise_exception`)."""
        if not self.chat_template:
            raise TokenizerError("the checkpoint has no tokenizer.chat_template")
        import jinja2
        import jinja2.sandbox

        def raise_exception(msg):
            raise TokenizerError(str(msg))
        env = jinja2.sandbox.ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
        env.globals["raise_exception"] = raise_exception
        bos = self.tokens[self.bos_token_id] if self.bos_token_id is not None else ""
        eos = self.tokens[self.eos_token_id] if self.eos_token_id is not None else ""
        return env.from_string(self.chat_template).render(messages=list(messages), bos_token=bos, eos_token=eos,
                                                          add_generation_prompt=add_generation_prompt)
