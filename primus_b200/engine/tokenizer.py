"""Tokenizer builder.

``build_tokenizer(tokenizer_type, tokenizer_model, vocab_size, make_vocab_size_divisible_by, tp)`` returns an
object with ``tokenize / detokenize / vocab_size / padded_vocab_size / eod / pad``.

Types (primus/backends/megatron/training/tokenizer/tokenizer.py:69-140 in the reference, which extends Megatron's
builder with Hugging Face aliases):

* ``NullTokenizer``   — mock data: text is a space-separated list of ids; ``eod = vocab_size`` (so the padded
  vocabulary is ``vocab_size + 1`` rounded up);
* ``HuggingFaceTokenizer`` and the model-named aliases (``Llama2Tokenizer``, ``Llama3Tokenizer``,
  ``DeepSeekV2Tokenizer``, ``DeepSeekV3Tokenizer``, ``Qwen2Tokenizer``, ``Qwen3Tokenizer``, ``MixtralTokenizer``)
  — ``transformers.AutoTokenizer`` on a local directory (no network access is attempted);
* ``SentencePieceTokenizer`` / ``GPTSentencePieceTokenizer`` — a ``.model`` file.
"""
from __future__ import annotations

from typing import List, Optional

HF_ALIASES = {"HuggingFaceTokenizer", "Llama2Tokenizer", "Llama3Tokenizer", "DeepSeekV2Tokenizer", "DeepSeekV3Tokenizer",
              "Qwen2Tokenizer", "Qwen3Tokenizer", "MixtralTokenizer", "GemmaTokenizer"}


def pad_vocab_size(vocab_size: int, divisible_by: int = 128, tp: int = 1) -> int:
    mult = divisible_by * tp
    return -(-vocab_size // mult) * mult


class _Base:
    def __init__(self, divisible_by: int, tp: int):
        self._div, self._tp = divisible_by, tp

    @property
    def padded_vocab_size(self) -> int:
        return pad_vocab_size(self.vocab_size, self._div, self._tp)


class NullTokenizer(_Base):
    def __init__(self, vocab_size: int, divisible_by: int = 128, tp: int = 1):
        super().__init__(divisible_by, tp)
        self._n = int(vocab_size)

    @property
    def vocab_size(self) -> int:
        return self._n + 1  # + eod

    @property
    def eod(self) -> int:
        return self._n

    pad = eod

    def tokenize(self, text: str) -> List[int]:
        return [int(t) for t in text.split()]

    def detokenize(self, ids) -> str:
        return " ".join(str(int(i)) for i in ids)


class HuggingFaceTokenizer(_Base):
    def __init__(self, path: str, divisible_by: int = 128, tp: int = 1, **kw):
        super().__init__(divisible_by, tp)
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(path, local_files_only=True, **kw)

    @property
    def vocab_size(self) -> int:
        return len(self.tok)

    @property
    def eod(self) -> int:
        return self.tok.eos_token_id

    @property
    def pad(self) -> int:
        return self.tok.pad_token_id if self.tok.pad_token_id is not None else self.tok.eos_token_id

    def tokenize(self, text: str) -> List[int]:
        return self.tok.encode(text, add_special_tokens=False)

    def detokenize(self, ids) -> str:
        return self.tok.decode(list(ids))

    def apply_chat_template(self, messages, **kw):
        return self.tok.apply_chat_template(messages, **kw)


class SentencePieceTokenizer(_Base):
    def __init__(self, model_file: str, divisible_by: int = 128, tp: int = 1):
        super().__init__(divisible_by, tp)
        import sentencepiece as spm

        self.sp = spm.SentencePieceProcessor(model_file=model_file)

    @property
    def vocab_size(self) -> int:
        return self.sp.get_piece_size()

    @property
    def eod(self) -> int:
        return self.sp.eos_id()

    @property
    def pad(self) -> int:
        return self.sp.pad_id() if self.sp.pad_id() >= 0 else self.sp.eos_id()

    def tokenize(self, text: str) -> List[int]:
        return self.sp.encode(text)

    def detokenize(self, ids) -> str:
        return self.sp.decode(list(ids))


def build_tokenizer(tokenizer_type: Optional[str], tokenizer_model: Optional[str] = None, vocab_size: Optional[int] = None,
                    make_vocab_size_divisible_by: int = 128, tp: int = 1):
    t = tokenizer_type or "NullTokenizer"
    if t == "NullTokenizer":
        return NullTokenizer(vocab_size if vocab_size is not None else 131072, make_vocab_size_divisible_by, tp)
    if t in HF_ALIASES:
        if not tokenizer_model:
            raise ValueError(f"{t} needs tokenizer_model (a local directory with the tokenizer files)")
        return HuggingFaceTokenizer(tokenizer_model, make_vocab_size_divisible_by, tp)
    if t in ("SentencePieceTokenizer", "GPTSentencePieceTokenizer"):
        if not tokenizer_model:
            raise ValueError(f"{t} needs tokenizer_model (a .model file)")
        return SentencePieceTokenizer(tokenizer_model, make_vocab_size_divisible_by, tp)
    raise ValueError(f"unknown tokenizer_type {t!r}")
