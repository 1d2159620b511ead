"""Tokenizers, chat templates, streaming tool-call parsers and the text generator (CPU)."""
import json

import pytest
import torch

from idrak_b200.generation import TextGenerator
from idrak_b200.models.decoder import build_decoder
from idrak_b200.models.spec import DecoderSpec
from idrak_b200.serve import GenerationOptions
from idrak_b200.text import (ByteTokenizer, ChatTemplate, create_parser, detect_format, load_tokenizer, render_chat,
                             tokenizer_from_gguf, train_tokenizer)

CORPUS = ["the quick brown fox jumps over the lazy dog", "pack my box with five dozen liquor jugs",
          "how vexingly quick daft zebras jump", "sphinx of black quartz judge my vow"] * 8


def test_byte_tokenizer_round_trip_and_streaming_utf8():
    t = ByteTokenizer()
    text = "héllo wörld ✓ 日本"
    ids = t.encode(text + "<|eos|>")
    assert ids[-1] == t.eos_token_ids[0] and t.decode(ids) == text
    assert t.decode(ids, skip_special_tokens=False).endswith("<|eos|>")
    s = t.stream()
    pieces = [s.push(i) for i in ids]
    assert "".join(pieces) + s.flush() == text and all("�" not in p for p in pieces)


@pytest.mark.parametrize("kind", ["bpe", "unigram", "wordpiece"])
def test_trained_tokenizers_round_trip(kind, tmp_path):
    specials = {"bpe": ["<|endoftext|>"], "unigram": ["<unk>", "</s>"], "wordpiece": ["[PAD]", "[SEP]"]}[kind]
    t = train_tokenizer(kind, CORPUS, 400 if kind == "bpe" else 120, specials)
    ids = t.encode("the quick zebras jump", add_special_tokens=False)
    assert len(ids) < len("the quick zebras jump") and t.decode(ids).replace(" ", "") == "thequickzebrasjump"
    assert t.eos_token_ids and t.vocab_size <= 400
    t.save(str(tmp_path / "tokenizer.json"))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps(
        {"eos_token": specials[-1], "chat_template": "{{ messages[0]['content'] }}!"}))
    again = load_tokenizer(str(tmp_path))
    assert again.encode("lazy dog", add_special_tokens=False) == t.encode("lazy dog", add_special_tokens=False)
    assert again.chat_template.endswith("!") and again.eos_token_ids == t.eos_token_ids


def test_tokenizer_from_gguf_metadata_matches_source():
    t = train_tokenizer("bpe", CORPUS, 300, ["<|endoftext|>"])
    model = json.loads(t.inner.to_str())["model"]
    vocab = sorted(model["vocab"].items(), key=lambda kv: kv[1])
    merges = [m if isinstance(m, str) else " ".join(m) for m in model["merges"]]
    meta = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": [k for k, _ in vocab],
            "tokenizer.ggml.token_type": [3 if k == "<|endoftext|>" else 1 for k, _ in vocab],
            "tokenizer.ggml.merges": merges, "tokenizer.ggml.eos_token_id": model["vocab"]["<|endoftext|>"]}
    g = tokenizer_from_gguf(meta)
    for s in CORPUS[:4] + ["jumps! over?"]:
        assert g.encode(s, False) == t.encode(s, False) and g.decode(g.encode(s, False)) == s
    assert g.eos_token_ids == (model["vocab"]["<|endoftext|>"],)


def test_chat_templates_render_and_refuse_foreign_parts():
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": [{"type": "text", "text": "hi"}]}]
    assert render_chat(msgs) == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    llama = ("{{ bos_token }}{% for m in messages %}{% if m['role'] not in ['user','system','assistant'] %}"
             "{{ raise_exception('bad role') }}{% endif %}[{{ m['role'] }}]{{ m['content'] | trim }}{% endfor %}"
             "{% if tools %}{{ tools | tojson }}{% endif %}")
    out = ChatTemplate(llama, bos_token="<s>").render(msgs, tools=[{"name": "f"}])
    assert out == '<s>[system]be brief[user]hi[{"name": "f"}]'
    with pytest.raises(ValueError, match="bad role"):
        render_chat([{"role": "tool", "content": "x"}], llama)
    with pytest.raises(ValueError, match="image_url"):
        render_chat([{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "x"}}]}])


def _run(parser, pieces):
    content, calls = "", []
    for p in pieces:
        d = parser.feed(p)
        content += d.content
        calls += d.tool_calls
    d = parser.finish()
    return content + d.content, calls + d.tool_calls


TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {}}}]


def test_tool_call_parsers_streaming():
    text = 'Let me check. <tool_call>{"name": "get_weather", "arguments": {"city": "Paris"}}</tool_call> done'
    for chunk in (1, 3, 7, len(text)):
        pieces = [text[i:i + chunk] for i in range(0, len(text), chunk)]
        content, calls = _run(create_parser("json", TOOLS), pieces)
        assert content == "Let me check.  done" and len(calls) == 1
        assert calls[0].name == "get_weather" and json.loads(calls[0].arguments) == {"city": "Paris"}
    # a marker look-alike and a body that does not parse stay text
    content, calls = _run(create_parser("json", TOOLS), ["a <tool", "box> b <tool_call>not json</tool_call>"])
    assert content == "a <toolbox> b <tool_call>not json</tool_call>" and calls == []
    # bare JSON answer: a call only when it names one of the request's tools
    content, calls = _run(create_parser("json", TOOLS), ['{"name": "get_weather", ', '"parameters": {"city": "Oslo"}}'])
    assert content == "" and json.loads(calls[0].arguments) == {"city": "Oslo"}
    content, calls = _run(create_parser("json", TOOLS), ['{"name": "other", "arguments": {}}'])
    assert calls == [] and content.startswith('{"name": "other"')
    content, calls = _run(create_parser("llama3", TOOLS), ['<|python_tag|>{"name": "get_weather", "parameters": {}}; '
                                                         '{"name": "get_weather", "parameters": {"city": "Rome"}}'])
    assert content == "" and len(calls) == 2
    content, calls = _run(create_parser("mistral", TOOLS), ['ok [TOOL_', 'CALLS][{"name": "get_weather", "arguments": {"a": 1}}]'])
    assert content == "ok " and calls[0].name == "get_weather"
    content, calls = _run(create_parser("pythonic", TOOLS), ['[get_weather(city="Lima", ', 'days=3)]'])
    assert content == "" and json.loads(calls[0].arguments) == {"city": "Lima", "days": 3}
    content, calls = _run(create_parser("pythonic", TOOLS), ["[1, 2, 3] is a list"])
    assert calls == [] and content == "[1, 2, 3] is a list"
    assert detect_format("...[TOOL_CALLS]...") == "mistral" and detect_format("<tool_call>") == "json"
    assert detect_format("{{ '<|python_tag|>' }}") == "llama3"
    with pytest.raises(KeyError, match="not registered"):
        create_parser("nope")


def test_failed_engine_step_wakes_callers_with_an_error():
    gen, m, tok = _generator()
    gen.start()
    try:
        def boom():
            raise ValueError("kernel refused")
        gen.engine._step = boom
        with pytest.raises(RuntimeError, match="kernel refused"):
            gen.generate("hello", GenerationOptions.greedy_options(4))
        assert not gen.engine.has_work()
    finally:
        gen.close()


def _generator(**kw):
    tok = ByteTokenizer()
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=tok.vocab_size, max_positions=256)
    m = build_decoder(spec, seed=3).float().eval()
    for p in m.parameters():
        p.data.mul_(3.0)
    return TextGenerator(m, tok, num_blocks=64, max_batch=4, **kw), m, tok


def test_text_generator_stream_equals_generate_and_stop_strings():
    gen, m, tok = _generator()
    o = GenerationOptions.greedy_options(24)
    full = gen.generate("hello", o)
    assert full.completion_tokens == 24 and full.finish_reason == "length" and full.prompt_tokens == 5
    assert "".join(gen.stream("hello", o)) == full.text
    visible = [c for c in full.text if c.isprintable()]
    if len(full.text) > 6:
        stop = full.text[4:6]
        cut = gen.generate("hello", GenerationOptions.greedy_options(24, stop=(stop,)))
        assert cut.finish_reason == "stop" and cut.text == full.text[: full.text.find(stop)]
    assert not gen.engine.has_work() and gen.engine.stats()["free_blocks"] == 64
    # batch (inline and with the background loop) equals one-by-one
    prompts = ["hello", "abc", "hello world"]
    single = [gen.generate(p, o).tokens for p in prompts]
    assert [r.tokens for r in gen.generate_batch(prompts, o)] == single
    gen.start()
    try:
        assert [r.tokens for r in gen.generate_batch(prompts, o)] == single
        r = gen.chat([{"role": "user", "content": "hi"}], o)
        assert r.prompt_tokens == 52 and 0 < r.completion_tokens <= 24 and r.finish_reason in ("stop", "length")
    finally:
        gen.close()
