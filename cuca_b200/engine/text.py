"""Text in and out, for model folders that bring a `tokenizer.json`.

The engine itself works on token ids. When the folder holds a Hugging Face `tokenizer.json`, it is read with the
`tokenizers` package (a tokenizer library, no model code) so that prompts may be strings, replies come with their
text, and stop strings can be honoured (`LocalModel::tokenize` and the text side of `generate` in the reference:
src/provider/local/mod.rs:3213-3276, which reads its vocabulary from the GGUF metadata instead).
"""
from __future__ import annotations

from pathlib import Path
from typing import List, Optional

_REPLACEMENT = "�"  # a byte-level vocabulary decodes half a character to this until the rest arrives


class TextCodec:
    def __init__(self, tokenizer):
        self._tok = tokenizer

    @classmethod
    def find(cls, model_dir: Optional[Path]) -> Optional["TextCodec"]:
        """The folder's tokenizer, or None when it has none."""
        if model_dir is None:
            return None
        f = Path(model_dir) / "tokenizer.json"
        if not f.is_file():
            return None
        try:
            from tokenizers import Tokenizer
        except ImportError as e:  # pragma: no cover - the package is part of the environment
            raise RuntimeError(f"{f} needs the `tokenizers` package to be read: {e}") from e
        return cls(Tokenizer.from_file(str(f)))

    def encode(self, text: str) -> List[int]:
        return list(self._tok.encode(text, add_special_tokens=True).ids)

    def decode(self, ids) -> str:
        return self._tok.decode(list(ids), skip_special_tokens=True)


class TextStream:
    """Turns a growing list of token ids into text fragments: each call returns what the new ids added. A fragment
    that ends inside a multi-byte character is held until the character is whole."""

    def __init__(self, codec: TextCodec):
        self.codec = codec
        self.sent = ""

    def push(self, ids) -> str:
        text = self.codec.decode(ids)
        while text.endswith(_REPLACEMENT):
            text = text[:-1]
        if not text.startswith(self.sent):  # the decoder rewrote earlier text (merging spaces): keep what was sent
            return ""
        delta, self.sent = text[len(self.sent):], text
        return delta
