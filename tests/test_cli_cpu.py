"""The command line's text handling on the CPU: the BOS rule with a tokenizer, and prompts
without one (crates/braidinfer-runtime/src/generate.rs:479-489 is the rule's source)."""
import json

import pytest

from braidinfer_b200.engine.cli import TextCodec

tokenizers = pytest.importorskip("tokenizers")


def tiny_tokenizer(folder, add_bos=None):
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    vocab = {"<unk>": 0, "BOS": 1, "EOS": 2, "hello": 3, "world": 4, "again": 5}
    t = Tokenizer(WordLevel(vocab, unk_token="<unk>"))
    t.pre_tokenizer = Whitespace()
    t.save(str(folder / "tokenizer.json"))
    if add_bos is not None:
        (folder / "tokenizer_config.json").write_text(json.dumps({"add_bos_token": add_bos}))
    return str(folder)


def test_bos_is_put_first_unless_it_is_there_or_switched_off(tmp_path):
    c = TextCodec(tiny_tokenizer(tmp_path), 6, bos=1)
    assert c.encode("hello world") == [1, 3, 4]                 # prepended
    assert c.encode("BOS hello") == [1, 3]                      # already there: not doubled
    assert c.encode("") == [1]
    assert c.decode([3, 4, 5]) == "hello world again"
    on = tmp_path / "on"
    on.mkdir()
    assert TextCodec(tiny_tokenizer(on, add_bos=True), 6, bos=1).encode("hello") == [1, 3]
    off = tmp_path / "off"
    off.mkdir()
    assert TextCodec(tiny_tokenizer(off, add_bos=False), 6, bos=1).encode("hello") == [3]      # add_bos_token false
    none = tmp_path / "none"
    none.mkdir()
    assert TextCodec(tiny_tokenizer(none), 6, bos=None).encode("hello") == [3]                 # the model names no BOS


def test_without_a_tokenizer_the_prompt_is_ids_or_bytes(tmp_path):
    c = TextCodec(str(tmp_path), 300, bos=1)                    # a folder without tokenizer.json
    assert c.encode("1, 5, 17") == [1, 5, 17] and c.encode("7 8") == [7, 8]
    assert c.encode("Hi!") == [72, 105, 33]                     # UTF-8 bytes, taken as they are: no BOS is added
    assert TextCodec(None, 100, bos=None).encode("Hi!") == [72, 5, 33]      # folded into a small vocabulary
    assert c.decode([4, 2]) == "4 2"
