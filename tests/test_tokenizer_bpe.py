"""The engine's own BPE tokenizer against the Hugging Face `tokenizers` implementation on vocabularies trained in the test
(byte-level with the Qwen split pattern and special tokens; SentencePiece-style with byte fallback)."""
import json
import os

import pytest

tokenizers = pytest.importorskip("tokenizers")

QWEN_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")

CORPUS = [
    "The quick brown fox jumps over the lazy dog. It's 12:45pm, isn't it? We'll see...",
    "def fib(n):\n    return n if n < 2 else fib(n - 1) + fib(n - 2)\n\n\nprint(fib(10))",
    "Unicode: naïve café — 東京タワー, Привет мир, 😀 emoji 👍🏽 and   runs   of   spaces\t\ttabs",
    "numbers 1234567890 3.14159 1e-9 0xDEADBEEF; symbols !@#$%^&*()_+-=[]{}|;':\",./<>?",
] * 3

SAMPLES = CORPUS[:4] + [
    "", " ", "  leading and trailing  ", "a", "\n\n", "It'S DON'T we'Ve", "x<|im_end|>y<|im_start|>user\nhi<|im_end|>",
    "unseen: ßøæ ĳ ‰ 𝔘𝔫𝔦𝔠𝔬𝔡𝔢 ‍ zero-width", "mixed1234abc 5 6  7", "tab\tsep\r\nwindows\r\nlines",
]


def _train_byte_level(tmp_path):
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    tk = Tokenizer(models.BPE())
    tk.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(QWEN_PATTERN), behavior="isolated", invert=False),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tk.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=600, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    tk.train_from_iterator(CORPUS, trainer)
    path = str(tmp_path / "tokenizer.json")
    tk.save(path)
    return tk, path


def test_byte_level_bpe_matches_the_hugging_face_encoder(tmp_path):
    from r4dx_b200.runtime.bpe import BpeTokenizer
    hf, path = _train_byte_level(tmp_path)
    mine = BpeTokenizer(path)
    assert mine.byte_level and mine.vocab_size == hf.get_vocab_size()
    assert mine._native, "the native merge loop should be in use"
    # the native loop and the Python loop agree piece by piece
    import random
    rnd = random.Random(0)
    alphabet = "abcdefghij THE the quick 0123 \n\t.,'é東😀"
    for _ in range(300):
        piece = "".join(rnd.choice(alphabet) for _ in range(rnd.randrange(1, 24)))
        from r4dx_b200.runtime.bpe import _B2U
        symbols = [_B2U[b] for b in piece.encode("utf-8")]
        py = [mine.vocab[t] for t in mine._merge(list(symbols))]
        assert mine._merge_native([mine.vocab[t] for t in symbols]) == py, piece
    for s in SAMPLES:
        want = hf.encode(s, add_special_tokens=False).ids
        got = mine.encode(s)
        assert got == want, (s, got, want)
        assert mine.decode(got, skip_special=False) == s
    ids = mine.encode("a<|im_end|>b")
    assert mine.added["<|im_end|>"] in ids and mine.decode(ids) == "ab" and mine.decode(ids, skip_special=False) == "a<|im_end|>b"
    assert mine.added["<|im_end|>"] in mine.eos_ids
    # exact bytes per token: a multi-byte character split over tokens never yields replacement characters mid-stream
    from r4dx_b200.runtime.tokenizer import StreamDecoder
    ids = mine.encode("né 😀!")
    dec = StreamDecoder(mine)
    text = "".join(dec.feed(i) for i in ids) + dec.flush()
    assert text == "né 😀!" and "�" not in text


def test_byte_fallback_bpe_matches_the_hugging_face_encoder(tmp_path):
    from tokenizers import Tokenizer, decoders, models, normalizers, trainers
    from r4dx_b200.runtime.bpe import BpeTokenizer
    tk = Tokenizer(models.BPE(byte_fallback=True, unk_token="<unk>", fuse_unk=True))
    tk.normalizer = normalizers.Sequence([normalizers.Prepend("▁"), normalizers.Replace(" ", "▁")])
    tk.decoder = decoders.Sequence([decoders.Replace("▁", " "), decoders.ByteFallback(), decoders.Fuse(), decoders.Strip(" ", 1, 0)])
    alphabet = [f"<0x{b:02X}>" for b in range(256)]
    trainer = trainers.BpeTrainer(vocab_size=700, special_tokens=["<unk>", "<bos>", "<eos>"] + alphabet, show_progress=False)
    tk.train_from_iterator(CORPUS, trainer)
    path = str(tmp_path / "tokenizer.json")
    tk.save(path)
    mine = BpeTokenizer(path)
    assert not mine.byte_level and mine.byte_fallback and mine.prefix_space
    for s in ["The quick brown fox", "naïve café", "unseen ß ĳ 𝔘 chars", "two  spaces", "It's 12:45pm"]:
        want = tk.encode(s, add_special_tokens=False).ids
        got = mine.encode(s)
        assert got == want, (s, got, want)
        # (the trainer can only register the byte tokens as special tokens, so they are kept while decoding here)
        assert mine.decode(got, skip_special=False) == s


def test_loader_prefers_the_own_tokenizer(tmp_path):
    from r4dx_b200.runtime.bpe import BpeTokenizer
    from r4dx_b200.runtime.tokenizer import load_tokenizer
    _, path = _train_byte_level(tmp_path)
    json.dump({"eos_token_id": [1]}, open(os.path.join(os.path.dirname(path), "generation_config.json"), "w"))
    tk, tpl = load_tokenizer(os.path.dirname(path))
    assert isinstance(tk, BpeTokenizer) and 1 in tk.eos_ids
    assert "hello" in tpl.render([{"role": "user", "content": "hello"}])


def test_sentencepiece_style_text_is_cut_at_space_runs_without_changing_the_ids(tmp_path):
    """A vocabulary whose tokens carry the space marker only as a leading run: cutting the text before every run of markers
    gives the ids of whole-text BPE (and of the Hugging Face encoder)."""
    from tokenizers import Tokenizer
    from r4dx_b200.runtime.bpe import BpeTokenizer
    chars = ["▁", "a", "b", "c", "d", "e", "\n", "."]
    merges = [("▁", "a"), ("a", "b"), ("▁", "▁"), ("▁a", "b"), ("c", "d"), ("▁▁", "c"), ("ab", "cd"), ("▁", "c"), ("d", "e"), ("▁▁", "▁")]
    vocab = {c: i for i, c in enumerate(chars)}
    for a, b in merges:
        vocab.setdefault(a + b, len(vocab))
    spec = {"version": "1.0", "truncation": None, "padding": None, "added_tokens": [],
            "normalizer": {"type": "Replace", "pattern": {"String": " "}, "content": "▁"}, "pre_tokenizer": None,
            "post_processor": None, "decoder": None,
            "model": {"type": "BPE", "dropout": None, "unk_token": None, "continuing_subword_prefix": None,
                      "end_of_word_suffix": None, "fuse_unk": False, "byte_fallback": False, "ignore_merges": False,
                      "vocab": vocab, "merges": [[a, b] for a, b in merges]}}
    path = str(tmp_path / "tokenizer.json")
    json.dump(spec, open(path, "w"))
    hf = Tokenizer.from_file(path)
    mine = BpeTokenizer(path)
    assert mine._sp_split and not mine.byte_level
    whole = BpeTokenizer(path)
    whole._sp_split = False
    for s in ["ab abcd  cde", "  c   ab", "a\nb. ab", "abcd", "   ", " a b c d e "]:
        want = hf.encode(s, add_special_tokens=False).ids
        assert mine.encode(s) == want == whole.encode(s), s
        assert mine.decode(mine.encode(s)) == s
