"""Instruct (chat) templates per model family and the streaming decoders built on them.

A template renders a role message into tokens (`render`), emits the assistant cue (`cue`), the
turn terminator (`seal`), knows the stop tokens, how tool definitions and tool results are
written (`equip`, `answer`) and how to split reasoning from the answer. Decoders consume
generated tokens incrementally and emit events (chat text deltas, reasoning segments, tool
calls). Families: llama3, llama2, qwen (ChatML: Qwen2/Qwen3), mistral, mistral3, gemma 2/3, gemma4,
phi3, olmo2, olmo3,
gpt-oss (harmony), kimi, deepseek-r1 style reasoning. Counterpart of runtime/src/model/instruct.rs and instruct/*.rs.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence


class Instruct:
    """Base: plain concatenation, no special tokens."""

    name = "plain"
    bos = ""
    stop_strings: Sequence[str] = ()
    think_open, think_close = "<think>", "</think>"
    tool_open, tool_close = "<tool_call>", "</tool_call>"
    drop_strings: Sequence[str] = ()      # framing the model writes around its answer; decoders swallow it
    fold_system = False                   # no system role: the system text opens the first user turn
    tool_role = "tool"                    # role under which tool results are rendered

    def format(self, role: str, message: str, first: bool) -> str:
        return message

    def cue_text(self) -> str:
        return ""

    def seal_text(self) -> str:
        return ""

    # ---- token level
    def render(self, role: str, message: str, tok, first: bool = False) -> List[int]:
        text = (self.bos if first else "") + self.format(role, message, first)
        return tok.encode(text)

    def cue(self, tok) -> List[int]:
        return tok.encode(self.cue_text())

    def seal(self, tok) -> List[int]:
        return tok.encode(self.seal_text())

    def stop_tokens(self, tok) -> List[int]:
        out = list(getattr(tok, "eos_tokens", []))
        for s in self.stop_strings:
            ids = tok.encode(s)
            if len(ids) == 1:
                out.append(ids[0])
        return sorted(set(out))

    # ---- tools
    def equip(self, tools: Sequence[dict]) -> str:
        """System-prompt text that declares the callable tools (JSON schema per tool)."""
        lines = ["You may call these tools. To call one, answer with "
                 f"{self.tool_open}{{\"name\": ..., \"arguments\": {{...}}}}{self.tool_close}.", ""]
        lines += [json.dumps(t) for t in tools]
        return "\n".join(lines)

    def answer(self, name: str, result: str) -> str:
        """Text of a tool result fed back to the model."""
        return json.dumps({"tool": name, "result": result})

    def tool_grammar(self, tools: Sequence[dict]) -> str:
        """EBNF of one tool call `{"name": <tool>, "arguments": {...}}`; the arguments follow the
        tool's `parameters` JSON schema when it has one, else any JSON object."""
        from .structured import JSON_RULES, json_schema_rules
        alts, rules = [], []
        for i, t in enumerate(tools):
            schema = t.get("parameters") or t.get("inputSchema")
            if isinstance(schema, dict) and schema.get("properties"):
                root, text = json_schema_rules(schema, f"t{i}x")
                rules.append(text)
            else:
                root = "object"
            alts.append(f'( {json.dumps(json.dumps(t["name"]))} ws "," ws "\\"arguments\\"" ws ":" ws {root} )')
        if not alts:
            alts = ['( "\\"none\\"" ws "," ws "\\"arguments\\"" ws ":" ws object )']
        return ('root ::= "{" ws "\\"name\\"" ws ":" ws call ws "}"\n' + "call ::= " + " | ".join(alts) + "\n"
                + "".join(rules) + JSON_RULES)


JSON_EBNF_TAIL = r'''object ::= "{" ws (pair (ws "," ws pair)*)? ws "}"
pair ::= string ws ":" ws value
array ::= "[" ws (value (ws "," ws value)*)? ws "]"
value ::= object | array | string | number | "true" | "false" | "null"
string ::= "\"" char* "\""
char ::= [^"\\] | "\\" ["\\/bfnrt]
number ::= "-"? [0-9]+ ("." [0-9]+)? ([eE] [+-]? [0-9]+)?
ws ::= [ \t\n]*
'''


class Llama3(Instruct):
    name = "llama3"
    bos = "<|begin_of_text|>"
    stop_strings = ("<|eot_id|>", "<|end_of_text|>")
    tool_open, tool_close = "<|python_tag|>", "<|eom_id|>"

    def format(self, role, message, first):
        return f"<|start_header_id|>{role}<|end_header_id|>\n\n{message}<|eot_id|>"

    def cue_text(self):
        return "<|start_header_id|>assistant<|end_header_id|>\n\n"

    def seal_text(self):
        return "<|eot_id|>"


class Llama2(Instruct):
    name = "llama2"
    bos = "<s>"
    stop_strings = ("</s>",)

    def __init__(self):
        self._system = ""

    def format(self, role, message, first):
        if role == "system":
            self._system = message
            return ""
        if role == "user":
            sys = f"<<SYS>>\n{self._system}\n<</SYS>>\n\n" if self._system else ""
            self._system = ""
            return f"[INST] {sys}{message} [/INST]"
        return f" {message} </s><s>"

    def seal_text(self):
        return " </s>"


class ChatML(Instruct):
    """Qwen2 / Qwen3 ChatML."""
    name = "qwen"
    stop_strings = ("<|im_end|>", "<|endoftext|>")

    def format(self, role, message, first):
        return f"<|im_start|>{role}\n{message}<|im_end|>\n"

    def cue_text(self):
        return "<|im_start|>assistant\n"

    def seal_text(self):
        return "<|im_end|>\n"

    def answer(self, name, result):
        return f"<tool_response>\n{result}\n</tool_response>"


class Mistral(Instruct):
    name = "mistral"
    bos = "<s>"
    stop_strings = ("</s>",)
    tool_open, tool_close = "[TOOL_CALLS]", "</s>"

    def format(self, role, message, first):
        if role in ("system", "user"):
            return f"[INST] {message} [/INST]"
        return f"{message}</s>"

    def seal_text(self):
        return "</s>"


class Gemma(Instruct):
    """Gemma 2 / 3: `<start_of_turn>role\n...<end_of_turn>\n`, roles user / model. There is no system
    role: a leading system message is written as the head of the first user turn
    (`<bos><start_of_turn>user\n{system}\n{user}<end_of_turn>\n`; model/instruct/gemma3.rs:1-8)."""
    name = "gemma"
    bos = "<bos>"
    stop_strings = ("<end_of_turn>", "<eos>")
    fold_system = True

    def format(self, role, message, first):
        role = "model" if role == "assistant" else "user"
        return f"<start_of_turn>{role}\n{message}<end_of_turn>\n"

    def cue_text(self):
        return "<start_of_turn>model\n"

    def seal_text(self):
        return "<end_of_turn>\n"


class Gemma4(Instruct):
    """Gemma 4: single-token turn delimiters `<|turn>` / `<turn|>` and a native system turn
    (`<bos><|turn>system\n{system}<turn|>\n<|turn>user\n{user}<turn|>\n<|turn>model\n`;
    model/instruct/gemma4.rs:1-9)."""
    name = "gemma4"
    bos = "<bos>"
    stop_strings = ("<turn|>", "<eos>")

    def format(self, role, message, first):
        role = {"assistant": "model", "tool": "user"}.get(role, role)
        return f"<|turn>{role}\n{message}<turn|>\n"

    def cue_text(self):
        return "<|turn>model\n"

    def seal_text(self):
        return "<turn|>\n"


class Mistral3(Instruct):
    """Mistral V3 template: `[SYSTEM_PROMPT]..[/SYSTEM_PROMPT]`, `[INST]..[/INST]`,
    `[AVAILABLE_TOOLS]..[/AVAILABLE_TOOLS]`, calls as `[TOOL_CALLS]name[ARGS]{json}`, results as
    `[TOOL_RESULTS]..[/TOOL_RESULTS]` (model/instruct/mistral3.rs:1-10)."""
    name = "mistral3"
    bos = "<s>"
    stop_strings = ("</s>",)
    tool_open, tool_close = "[TOOL_CALLS]", "</s>"

    def format(self, role, message, first):
        if role == "system":
            return f"[SYSTEM_PROMPT]{message}[/SYSTEM_PROMPT]"
        if role == "user":
            return f"[INST]{message}[/INST]"
        if role == "tool":
            return f"[TOOL_RESULTS]{message}[/TOOL_RESULTS]"
        return f"{message}</s>"

    def seal_text(self):
        return "</s>"

    def equip(self, tools):
        return "[AVAILABLE_TOOLS]" + json.dumps([{"type": "function", "function": t} for t in tools]) + "[/AVAILABLE_TOOLS]"

    def answer(self, name, result):
        return f"[TOOL_RESULTS]{result}[/TOOL_RESULTS]"

    def parse_tool_call(self, text: str):
        """`name[ARGS]{json}` (the body after `[TOOL_CALLS]`) -> (name, arguments)."""
        name, sep, args = text.partition("[ARGS]")
        if not sep:
            return None
        try:
            return name.strip(), json.loads(args)
        except json.JSONDecodeError:
            return None


class Olmo2(Instruct):
    """OLMo 2: `<|endoftext|>` opens the chat and ends an assistant turn; plain `<|system|>` / `<|user|>` /
    `<|assistant|>` markers on their own line, messages separated by newlines
    (model/instruct/olmo2.rs:5-16)."""
    name = "olmo2"
    bos = "<|endoftext|>"
    stop_strings = ("<|endoftext|>",)

    def format(self, role, message, first):
        if role == "assistant":
            return f"<|assistant|>\n{message}<|endoftext|>"
        return f"<|{'user' if role == 'tool' else role}|>\n{message}\n"

    def cue_text(self):
        return "<|assistant|>\n"

    def seal_text(self):
        return "<|endoftext|>"


class Olmo3(Instruct):
    """OLMo 3: ChatML turns; tool definitions ride in the system turn inside `<functions>..</functions>`,
    calls come back as `<function_calls>..</function_calls>`, results go in an `environment` turn and the
    assistant cue opens a `<think>` block (model/instruct/olmo3.rs:4-8)."""
    name = "olmo3"
    stop_strings = ("<|im_end|>", "<|endoftext|>")
    tool_open, tool_close = "<function_calls>", "</function_calls>"
    tool_role = "environment"

    def format(self, role, message, first):
        role = "environment" if role == "tool" else role
        return f"<|im_start|>{role}\n{message}<|im_end|>\n"

    def cue_text(self):
        return "<|im_start|>assistant\n<think>"

    def seal_text(self):
        return "<|im_end|>\n"

    def equip(self, tools):
        return "<functions>" + "\n".join(json.dumps(t) for t in tools) + "</functions>"

    def answer(self, name, result):
        return result


class Phi3(Instruct):
    name = "phi3"
    stop_strings = ("<|end|>", "<|endoftext|>")

    def format(self, role, message, first):
        return f"<|{role}|>\n{message}<|end|>\n"

    def cue_text(self):
        return "<|assistant|>\n"

    def seal_text(self):
        return "<|end|>\n"


class GptOss(Instruct):
    """Harmony format of GPT-OSS: `<|start|>role<|message|>text<|end|>`; the assistant writes its
    reasoning on the `analysis` channel, tool calls on `commentary` (ended by `<|call|>`) and the
    answer on `final` (ended by `<|return|>`)."""
    name = "gptoss"
    stop_strings = ("<|return|>", "<|call|>")
    think_open, think_close = "<|channel|>analysis<|message|>", "<|end|>"
    tool_open, tool_close = "<|constrain|>json<|message|>", "<|call|>"
    drop_strings = ("<|start|>assistant", "<|channel|>final<|message|>", "<|end|>", "<|return|>")

    def format(self, role, message, first):
        if role == "assistant":
            return f"<|start|>assistant<|channel|>final<|message|>{message}<|end|>"
        if role == "tool":
            return f"<|start|>functions<|message|>{message}<|end|>"
        return f"<|start|>{'developer' if role == 'system' and not first else role}<|message|>{message}<|end|>"

    def cue_text(self):
        return "<|start|>assistant"

    def seal_text(self):
        return "<|return|>"

    def equip(self, tools):
        lines = ["# Tools", "", "## functions", "", "namespace functions {", ""]
        for t in tools:
            lines += [f"// {t.get('description', '')}",
                      f"type {t['name']} = (_: {json.dumps(t.get('parameters') or t.get('inputSchema') or {})}) => any;", ""]
        lines += ["} // namespace functions", "",
                  "Call a tool with <|channel|>commentary to=functions.NAME <|constrain|>json<|message|>{...}<|call|>."]
        return "\n".join(lines)

    def answer(self, name, result):
        return f"<|start|>functions.{name} to=assistant<|channel|>commentary<|message|>{result}<|end|>"


class Kimi(Instruct):
    """Kimi-K2 turns: `<|im_system|>`, `<|im_user|>`, `<|im_assistant|>` headers closed by `<|im_middle|>`."""
    name = "kimi"
    stop_strings = ("<|im_end|>",)
    tool_open, tool_close = "<|tool_call_argument_begin|>", "<|tool_call_end|>"

    def format(self, role, message, first):
        tag = {"system": "<|im_system|>", "user": "<|im_user|>", "assistant": "<|im_assistant|>"}.get(role, "<|im_system|>")
        return f"{tag}{role}<|im_middle|>{message}<|im_end|>"

    def cue_text(self):
        return "<|im_assistant|>assistant<|im_middle|>"

    def seal_text(self):
        return "<|im_end|>"


class R1(ChatML):
    """DeepSeek-R1 style: the assistant cue opens a reasoning block."""
    name = "r1"

    def cue_text(self):
        return "<|im_start|>assistant\n<think>\n"


FAMILIES: Dict[str, type] = {"llama3": Llama3, "llama": Llama3, "llama2": Llama2, "qwen": ChatML, "qwen2": ChatML,
                             "qwen3": ChatML, "qwen3_moe": ChatML, "olmo2": Olmo2, "olmo3": Olmo3,
                             "mistral": Mistral, "mistral3": Mistral3, "mixtral": Mistral, "gemma": Gemma,
                             "gemma2": Gemma, "gemma3": Gemma, "gemma3n": Gemma, "gemma4": Gemma4, "phi3": Phi3, "r1": R1, "gpt_oss": GptOss,
                             "gptoss": GptOss, "kimi": Kimi, "plain": Instruct}


def for_arch(arch: str) -> Instruct:
    return FAMILIES.get(arch, Instruct)()


# ------------------------------------------------------------------------------ streaming decoders
@dataclass
class Event:
    kind: str                  # delta | done | thinking | thinking_done | tool_call
    text: str = ""
    call: Optional[dict] = None


class ChatDecoder:
    """Feeds generated tokens, yields printable text deltas; `done` at a stop token. Incomplete
    UTF-8 sequences are held back until they complete."""

    def __init__(self, tok, instruct: Instruct):
        self.tok, self.stop = tok, set(instruct.stop_tokens(tok))
        self.ids: List[int] = []
        self.emitted = ""
        self.finished = False

    def feed(self, tokens: Sequence[int]) -> List[Event]:
        out = []
        for t in tokens:
            if self.finished:
                break
            if t in self.stop:
                self.finished = True
                out.append(Event("done", self.emitted))
                break
            self.ids.append(t)
            text = self.tok.decode(self.ids)
            if text.endswith("�"):
                continue
            if len(text) > len(self.emitted):
                out.append(Event("delta", text[len(self.emitted):]))
                self.emitted = text
        return out


class ReasoningDecoder:
    """Splits `<think>...</think>` from the answer in a text stream."""

    def __init__(self, instruct: Instruct, starts_in_think: bool = False):
        self.open, self.close = instruct.think_open, instruct.think_close
        self.drops = tuple(instruct.drop_strings)
        self.in_think = starts_in_think
        self.buf = ""

    def feed(self, text: str) -> List[Event]:
        self.buf += text
        out = []
        while True:
            # inside a reasoning block only its end matters; outside, its start and the framing to swallow
            tags = (self.close,) if self.in_think else (self.open,) + self.drops
            hits = [(self.buf.find(t), -len(t), t) for t in tags if t and self.buf.find(t) >= 0]
            if not hits:
                keep = max(0, len(self.buf) - max(len(t) for t in tags) + 1)     # a tag may be split across deltas
                if keep:
                    out.append(Event("thinking" if self.in_think else "delta", self.buf[:keep]))
                    self.buf = self.buf[keep:]
                break
            i, _, tag = min(hits)        # earliest; the longer tag on a tie
            if i:
                out.append(Event("thinking" if self.in_think else "delta", self.buf[:i]))
            self.buf = self.buf[i + len(tag):]
            if self.in_think:
                out.append(Event("thinking_done"))
                self.in_think = False
            elif tag == self.open:
                self.in_think = True
        return out

    def flush(self) -> List[Event]:
        out = [Event("thinking" if self.in_think else "delta", self.buf)] if self.buf else []
        self.buf = ""
        return out


class ToolDecoder:
    """Extracts tool calls (`<tool_call>{json}</tool_call>` or the family's tags) from a text stream."""

    def __init__(self, instruct: Instruct):
        self.open, self.close = instruct.tool_open, instruct.tool_close
        self.buf = ""

    def feed(self, text: str) -> List[Event]:
        self.buf += text
        out = []
        while True:
            i = self.buf.find(self.open)
            if i < 0:
                break
            j = self.buf.find(self.close, i + len(self.open))
            if j < 0:
                break
            body = self.buf[i + len(self.open):j].strip()
            try:
                call = json.loads(body)
                out.append(Event("tool_call", body, call))
            except json.JSONDecodeError:
                out.append(Event("delta", self.buf[i:j + len(self.close)]))
            self.buf = self.buf[:i] + self.buf[j + len(self.close):]
        return out
