"""The command line's text path: the small byte-pair tokenizer read from a
tokenizer.json the test writes (encode, decode, merges by rank, the space marker),
and `llmgen -prompt` end to end on the GPU with the cache options.  The rules are
the reference's (loader/tokenizer/tokenizer.go:92-188)."""
import json
import os
import subprocess
import sys

import pytest

from go_tinygrad_b200.cli.llmgen import parser
from go_tinygrad_b200.cli.tokenizer import Tokenizer
from conftest import ROOT, TINY

# A dozen entries: single characters, two merged pieces, two whole words with the
# byte-level space marker, one added token.
VOCAB = {"h": 0, "e": 1, "l": 2, "o": 3, "w": 4, "r": 5, "d": 6, "he": 7, "ll": 8, "hell": 9,
         "Ġworld": 10, "Ġ": 11, "hello": 12, "Ġwor": 13}
MERGES = ["h e", "l l", "he ll", "Ġ w"]           # rank = position: "h e" merges first


def write_tokenizer(folder, vocab=VOCAB, merges=MERGES):
    doc = {"model": {"type": "BPE", "vocab": vocab, "merges": merges},
           "added_tokens": [{"id": 14, "content": "<|endoftext|>"}]}
    path = os.path.join(folder, "tokenizer.json")
    with open(path, "w", encoding="utf-8") as f:
        json.dump(doc, f, ensure_ascii=False)
    return path


def test_encode_whole_words_merges_by_rank_and_decode(tmp_path):
    tok = Tokenizer(write_tokenizer(str(tmp_path)))
    assert tok.marker == "Ġ"
    # "hello" and "Ġworld" are in the vocabulary whole: one token each (direct lookup first)
    assert tok.encode("hello world") == [12, 10]
    assert tok.decode([12, 10]) == "hello world"
    # "hellow" is not: characters, merged by rank: h e -> he, l l -> ll, he ll -> hell; o and w stay
    assert tok.encode("hellow") == [9, 3, 4]
    # a second word gets the marker in front; "Ġwo" has no merge beyond "Ġ w", whose result is no
    # vocabulary entry and is dropped, as the reference drops pieces it does not know; "o" stays
    assert tok.encode("he wo") == [7, 3]
    # runs of whitespace separate words and leave nothing behind
    assert tok.encode("  hello \n world ") == [12, 10]
    assert tok.decode(tok.encode("hello world")) == "hello world"
    assert tok.decode([14, 99]) == "<|endoftext|>"     # an added token; an unknown id is skipped
    assert tok.encode("") == []


def test_sentencepiece_marker_is_detected(tmp_path):
    vocab = {"▁the": 0, "the": 1, "▁cat": 2, "cat": 3}
    tok = Tokenizer(write_tokenizer(str(tmp_path), vocab, []))
    assert tok.marker == "▁"
    assert tok.encode("the cat") == [1, 2]
    assert tok.decode([1, 2]) == "the cat"


def test_command_line_options_keep_the_reference_names():
    # cmd/llmgen/main.go:15-28: -model, -prompt, -tokens (50), -gpu, -gpu-layers (0 = all)
    args = parser().parse_args(["-model", "m", "-prompt", "hi", "-tokens", "7", "-gpu", "-max-len", "128", "-slots", "3"])
    assert (args.model, args.prompt, args.tokens, args.gpu, args.gpu_layers) == ("m", "hi", 7, True, 0)
    assert (args.max_len, args.slots) == (128, 3)
    assert parser().parse_args(["-model", "m"]).tokens == 50
    assert parser().parse_args(["-model", "m", "-max-batch", "5"]).slots == 5


@pytest.mark.gpu
def test_llmgen_takes_a_text_prompt_and_cache_options(tmp_path):
    import go_tinygrad_b200 as lib
    import plain_llama
    folder = str(tmp_path / "model")
    lib.write_random_model(folder, TINY["A"], seed=4, dtype="bfloat16", std=0.12, norm_std=0.05)
    write_tokenizer(folder)
    cfg, w = plain_llama.read_model(folder)
    prompt = [12, 10]                                    # "hello world"
    want = plain_llama.generate(cfg, w, prompt, 6)
    run = lambda *extra: subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "llmgen"), "-model", folder, "-prompt", "hello world",
         "-dtype", "float32", "-stop", "999", *extra], capture_output=True, text=True, timeout=300)
    out = run("-tokens", "6")
    assert out.returncode == 0, out.stderr
    assert "Prompt: 'hello world' (2 tokens)" in out.stdout
    assert f"[0] ids: {' '.join(map(str, want))}  (length)" in out.stdout
    assert "Generated tokens: 6" in out.stdout
    # a slot that holds 5 tokens: the prompt's two and three new ones fed back; the fourth new token
    # is sampled, has no position left to be fed at, and ends the sequence
    short = run("-tokens", "6", "-max-len", "5", "-slots", "1")
    assert short.returncode == 0, short.stderr
    assert f"[0] ids: {' '.join(map(str, want[:4]))}  (capacity)" in short.stdout
    # no tokenizer.json: a text prompt is refused with a pointer to -ids
    os.remove(os.path.join(folder, "tokenizer.json"))
    bad = run("-tokens", "2")
    assert bad.returncode == 1 and "-ids" in bad.stderr
