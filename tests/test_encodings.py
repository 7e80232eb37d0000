"""Chat framing goldens and tokenizer construction (CPU)."""
import json

from pocketllm_b200.encoding import chat, dsv4, gguf_tokenizer as gt


def test_dsv4_multi_turn_thinking_golden():
    msgs = [{"role": "system", "content": "You are a helpful assistant."},
            {"role": "user", "content": "Hello"},
            {"role": "assistant", "reasoning_content": "The user said hello, I should greet back.", "content": "Hi there! How can I help you?"},
            {"role": "user", "content": "What is the capital of France?"},
            {"role": "assistant", "reasoning_content": "The user asks about the capital of France. It is Paris.",
             "content": "The capital of France is Paris."}]
    want = ("<｜begin▁of▁sentence｜>You are a helpful assistant.<｜User｜>Hello<｜Assistant｜></think>Hi there! How can I help you?"
            "<｜end▁of▁sentence｜><｜User｜>What is the capital of France?<｜Assistant｜><think>The user asks about the capital of "
            "France. It is Paris.</think>The capital of France is Paris.<｜end▁of▁sentence｜>")
    assert dsv4.encode_messages(msgs, thinking_mode="thinking") == want


def test_dsv4_generation_prompt_and_modes():
    msgs = [{"role": "user", "content": [{"type": "text", "text": "2+2?"}]}]
    assert dsv4.encode_messages(msgs) == "<｜begin▁of▁sentence｜><｜User｜>2+2?<｜Assistant｜></think>"
    p = dsv4.encode_messages(msgs, thinking_mode="thinking", reasoning_effort="high")
    assert p.startswith("<｜begin▁of▁sentence｜>Reasoning Effort: Absolute maximum") and p.endswith("<｜Assistant｜><think>")
    assert dsv4.normalize_effort("medium") == "low"


def test_dsv4_tools_roundtrip():
    tools = [{"type": "function", "function": {"name": "get_weather", "description": "d",
                                               "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}}]
    call = [{"id": "x", "type": "function", "function": {"name": "get_weather", "arguments": json.dumps({"city": "Paris", "days": 3})}}]
    msgs = [{"role": "user", "content": "weather?"}, {"role": "assistant", "content": "", "tool_calls": call},
            {"role": "tool", "tool_call_id": "x", "content": "sunny"}]
    p = dsv4.encode_messages(msgs, tools=tools)
    assert "## Tools" in p and '<｜DSML｜invoke name="get_weather">' in p
    assert '<｜DSML｜parameter name="city" string="true">Paris</｜DSML｜parameter>' in p
    assert '<｜DSML｜parameter name="days" string="false">3</｜DSML｜parameter>' in p
    assert "<｜User｜><tool_result>sunny</tool_result><｜Assistant｜></think>" in p
    completion = "</think>Let me check.\n\n" + dsv4.render_tool_calls(call) + dsv4.EOS
    m = dsv4.parse_completion(completion)
    assert m["content"] == "Let me check."
    assert m["tool_calls"][0]["function"]["name"] == "get_weather"
    assert json.loads(m["tool_calls"][0]["function"]["arguments"]) == {"city": "Paris", "days": 3}
    t = dsv4.parse_completion("<think>hmm</think>answer", thinking_mode="thinking")
    assert t["reasoning_content"] == "hmm" and t["content"] == "answer"


def test_glm_and_minimax_framing():
    assert chat.render_glm("hi", system_prompt="S") == "[gMASK]<sop><|system|>\nS<|user|>\nhi<|assistant|>"
    assert chat.render_glm("hi", thinking=True).endswith("<|assistant|>\n<think>")
    mm = chat.render_minimax("hi", system_prompt="S")
    assert mm == "]~!b[]~b]system\nS[e~[\n]~b]user\nhi[e~[\n]~b]ai\n"
    assert chat.split_thinking("<think>a</think>\nb") == ("a", "b")


def test_gguf_bpe_tokenizer_from_metadata():
    # bytes-level vocab for a few ASCII symbols plus merges
    from tokenizers import pre_tokenizers
    alphabet = pre_tokenizers.ByteLevel.alphabet()
    base = sorted(alphabet)
    tokens = base + ["he", "ll", "hell", "hello", "<|eot|>"]
    md = {"general.architecture": "glm-dsa", "tokenizer.ggml.model": "gpt2", "tokenizer.ggml.pre": "glm4",
          "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.merges": ["h e", "l l", "he ll", "hell o"],
          "tokenizer.ggml.token_type": [1] * (len(tokens) - 1) + [3], "tokenizer.ggml.eos_token_id": len(tokens) - 1,
          "glm-dsa.context_length": 1024}
    tok = gt.build_tokenizer(md)
    ids = tok.encode("hello<|eot|>", add_special_tokens=False).ids
    assert ids == [tokens.index("hello"), len(tokens) - 1]
    assert gt.decode_ids(tok, ids[:1]) == "hello"
    assert gt.context_length(md) == 1024 and gt.special_ids(md)["eos"] == len(tokens) - 1
    # digits split into groups of at most three with the llama3-style pre-tokenizer
    assert len(tok.encode("1234567").tokens) >= 3
    assert gt.parse_ids_csv("1, 2\n3") == [1, 2, 3]
