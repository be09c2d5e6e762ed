"""Optional text front end: a thin wrapper over the tokenizer file beside a
checkpoint.  The library itself works on token ids; only the command line's
text prompt needs this.  As in gpt-fast (tokenizer.py:102-112) a model whose
name contains "llama-3" has a tiktoken vocabulary, every other one a
SentencePiece model."""
import os


class SentencePieceTokenizer:
    def __init__(self, path):
        import sentencepiece
        self._sp = sentencepiece.SentencePieceProcessor(model_file=str(path))

    def encode(self, text):
        return list(self._sp.encode(text))

    def decode(self, ids):
        return self._sp.decode(list(ids))

    def bos_id(self):
        return self._sp.bos_id()

    def eos_id(self):
        return self._sp.eos_id()


class TiktokenTokenizer:
    """Llama-3 vocabulary: the BPE ranks of the file, then 256 special tokens of
    which the first two are begin/end of text (gpt-fast tokenizer.py:49-84)."""
    SPLIT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*"
             r"|\s*[\r\n]+|\s+(?!\S)|\s+")
    N_SPECIAL = 256

    def __init__(self, path):
        import tiktoken
        from tiktoken.load import load_tiktoken_bpe
        ranks = load_tiktoken_bpe(str(path))
        names = ["<|begin_of_text|>", "<|end_of_text|>", "<|reserved_special_token_0|>", "<|reserved_special_token_1|>",
                 "<|reserved_special_token_2|>", "<|reserved_special_token_3|>", "<|start_header_id|>",
                 "<|end_header_id|>", "<|reserved_special_token_4|>", "<|eot_id|>"]
        names += [f"<|reserved_special_token_{i}|>" for i in range(5, self.N_SPECIAL - 5)]
        special = {n: len(ranks) + i for i, n in enumerate(names)}
        self._enc = tiktoken.Encoding(name=os.path.basename(str(path)), pat_str=self.SPLIT, mergeable_ranks=ranks,
                                      special_tokens=special)
        self._bos, self._eos = special["<|begin_of_text|>"], special["<|end_of_text|>"]

    def encode(self, text):
        return self._enc.encode(text)

    def decode(self, ids):
        return self._enc.decode(list(ids))

    def bos_id(self):
        return self._bos

    def eos_id(self):
        return self._eos


def get_tokenizer(path, model_name):
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no tokenizer file at {path}")
    return TiktokenTokenizer(path) if "llama-3" in str(model_name).lower() else SentencePieceTokenizer(path)
