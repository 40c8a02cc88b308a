"""Chat templates per family against the rendered strings the reference's template tests pin
(runtime/src/model/instruct/{olmo2,olmo3,mistral3,gemma3,gemma4}.rs)."""
import json

from pie_b200.runtime import instruct as I
from pie_b200.runtime.tokenizer import ByteTokenizer

TOK = ByteTokenizer()


def chat(ins, turns, cue=True):
    out = ""
    for i, (role, msg) in enumerate(turns):
        out += TOK.decode(ins.render(role, msg, TOK, first=i == 0))
    return out + (TOK.decode(ins.cue(TOK)) if cue else "")


def test_olmo3_multi_turn_and_environment_turn():
    ins = I.for_arch("olmo3")
    got = chat(ins, [("system", "Hello"), ("user", "Hello"), ("assistant", "Hello"), ("user", "Hello")])
    assert got == ("<|im_start|>system\nHello<|im_end|>\n<|im_start|>user\nHello<|im_end|>\n"
                   "<|im_start|>assistant\nHello<|im_end|>\n<|im_start|>user\nHello<|im_end|>\n"
                   "<|im_start|>assistant\n<think>")
    assert ins.format("tool", "Hello", False) == "<|im_start|>environment\nHello<|im_end|>\n"
    tools = ins.equip([{"name": "f", "parameters": {}}])
    assert tools.startswith("<functions>") and tools.endswith("</functions>") and json.loads(tools[11:-12])["name"] == "f"
    assert (ins.tool_open, ins.tool_close) == ("<function_calls>", "</function_calls>")


def test_olmo2_plain_role_markers():
    ins = I.for_arch("olmo2")
    got = chat(ins, [("system", "S"), ("user", "U"), ("assistant", "A"), ("user", "U2")])
    assert got == "<|endoftext|><|system|>\nS\n<|user|>\nU\n<|assistant|>\nA<|endoftext|><|user|>\nU2\n<|assistant|>\n"
    assert "<|endoftext|>" in ins.stop_strings and "<|end|>" not in got


def test_mistral3_blocks_and_tool_syntax():
    ins = I.for_arch("mistral3")
    got = chat(ins, [("system", "S"), ("user", "U"), ("assistant", "A"), ("tool", "42")], cue=False)
    assert got == "<s>[SYSTEM_PROMPT]S[/SYSTEM_PROMPT][INST]U[/INST]A</s>[TOOL_RESULTS]42[/TOOL_RESULTS]"
    eq = ins.equip([{"name": "add", "parameters": {"type": "object"}}])
    assert eq.startswith("[AVAILABLE_TOOLS][") and eq.endswith("][/AVAILABLE_TOOLS]")
    assert ins.parse_tool_call('add[ARGS]{"a": 1}') == ("add", {"a": 1})
    assert ins.parse_tool_call("no call") is None
    assert I.for_arch("mistral").format("user", "U", True) == "[INST] U [/INST]"     # the older template is kept


def test_gemma4_turn_tokens_and_native_system():
    ins = I.for_arch("gemma4")
    got = chat(ins, [("system", "S"), ("user", "U")])
    assert got == "<bos><|turn>system\nS<turn|>\n<|turn>user\nU<turn|>\n<|turn>model\n"


def test_gemma3_folds_system_into_first_user_turn_through_the_context():
    from test_runtime_cpu import CounterBehavior, MockDriver, engine_with
    from pie_b200.sdk import Context, Model
    eng = engine_with(MockDriver(CounterBehavior(), total_pages=32))
    try:
        entry = eng.models["mock"]
        entry.tokenizer, entry.instruct = ByteTokenizer(), I.for_arch("gemma3")

        async def prog(args):
            m = Model.load("mock")
            c = Context(m).system("S").user("U").cue()
            a = TOK.decode(c.buffer)
            c.release()
            c2 = Context(m).system("only").cue()
            b = TOK.decode(c2.buffer)
            c2.release()
            return json.dumps([a, b])
        eng.register_program("t", prog)
        a, b = json.loads(eng.run("t", {}, 30))
    finally:
        eng.shutdown()
    assert a == "<bos><start_of_turn>user\nS\nU<end_of_turn>\n<start_of_turn>model\n"
    assert b == "<bos><start_of_turn>user\nonly<end_of_turn>\n<start_of_turn>model\n"


def test_python_example_inferlet_streams_answer_and_keeps_reasoning_apart():
    """The walk-through inferlet on a chat model: tokens go through the chat decoder and the reasoning decoder; what is inside
    the think tags does not reach the answer. The scripted driver speaks a reply with a reasoning block."""
    from test_runtime_cpu import MockDriver, engine_with
    from pie_b200.driver.mock import ScriptedBehavior
    from pie_b200.inferlets import install_all
    ins = I.for_arch("qwen3")
    reply = TOK.encode("<think>hm</think>Paris.")
    eng = engine_with(MockDriver(ScriptedBehavior(reply + TOK.encode("!")), total_pages=64))
    try:
        entry = eng.models["mock"]
        entry.tokenizer, entry.instruct = TOK, ins
        entry.inference.cohorts = []
        install_all(eng)
        out = eng.run("python-example", {"max_tokens": len(reply) + 3}, 60)
    finally:
        eng.shutdown()
    assert out.startswith("Paris.") and out.rstrip("!") == "Paris." and "hm" not in out and "think" not in out
