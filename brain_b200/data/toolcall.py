"""Synthetic tool-calling task (reference: crates/data/src/toolcall.rs — a catalogue of small tool
schemas, a user request that determines exactly one call, scoring by call name + argument
equality with number/string leniency)."""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Dict, List, Optional

from .chat import ChatExample, parse_tool_calls
from .rng import Rng

_CATALOGUE = [
    ("get_weather", "Get the current weather for a city.", [("city", "string", "City name")],
     "What is the weather in {city}?", {"city": ["Paris", "Oslo", "Lima", "Cairo", "Tokyo", "Quito"]}),
    ("add_numbers", "Add two numbers.", [("a", "number", "First addend"), ("b", "number", "Second addend")],
     "Please add {a} and {b}.", {"a": list(range(1, 60)), "b": list(range(1, 60))}),
    ("set_timer", "Start a countdown timer.", [("minutes", "number", "Length in minutes")],
     "Set a timer for {minutes} minutes.", {"minutes": [1, 2, 3, 5, 10, 15, 20, 30, 45]}),
    ("translate", "Translate a word to a language.", [("word", "string", "Word"), ("language", "string", "Target language")],
     "Translate '{word}' into {language}.", {"word": ["cat", "house", "tree", "water", "sun"],
                                            "language": ["French", "German", "Spanish", "Swedish"]}),
    ("lookup_stock", "Look up a stock price by ticker.", [("ticker", "string", "Ticker symbol")],
     "How is {ticker} trading?", {"ticker": ["ACME", "GLOB", "INIT", "ZETA", "ORCA"]}),
    ("send_message", "Send a short message to a contact.", [("to", "string", "Recipient"), ("body", "string", "Text")],
     "Tell {to}: {body}", {"to": ["Ana", "Bo", "Chen", "Dee"], "body": ["running late", "call me", "all done", "see you at 5"]}),
]


def schema(name, desc, params) -> Dict:
    return {"type": "function", "function": {
        "name": name, "description": desc,
        "parameters": {"type": "object",
                       "properties": {p: {"type": t, "description": d} for p, t, d in params},
                       "required": [p for p, _, _ in params]}}}


def system_prompt(tools: List[Dict]) -> str:
    lines = "\n".join(json.dumps(t) for t in tools)
    return ("# Tools\n\nYou may call one function to assist with the user query.\n\n"
            "You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n"
            f"{lines}\n</tools>\n\nFor each function call, return a json object with function name "
            "and arguments within <tool_call></tool_call> XML tags.")


@dataclass
class ToolCase:
    tools: List[Dict]
    user: str
    name: str
    arguments: Dict

    def response_str(self) -> str:
        return f'<tool_call>\n{{"name": "{self.name}", "arguments": {json.dumps(self.arguments)}}}\n</tool_call>'

    def to_chat_example(self) -> ChatExample:
        return ChatExample(self.user, self.response_str(), system_prompt(self.tools))


def generate(n: int, n_tools: int, seed: int) -> List[ToolCase]:
    rng = Rng(seed)
    out = []
    k = max(1, min(n_tools, len(_CATALOGUE)))
    for _ in range(n):
        order = list(range(len(_CATALOGUE)))
        for i in range(len(order) - 1, 0, -1):          # Fisher-Yates with the shared RNG
            j = rng.gen_range_inclusive(0, i)
            order[i], order[j] = order[j], order[i]
        picks = [_CATALOGUE[i] for i in order[:k]]
        name, desc, params, template, values = picks[rng.gen_range_inclusive(0, k - 1)]
        args = {p: rng.choice(values[p]) for p, _, _ in params}
        out.append(ToolCase([schema(a, b, c) for a, b, c, _, _ in picks], template.format(**args), name, args))
    return out


def _val_eq(a, b) -> bool:
    num = (int, float)
    if isinstance(a, str) and isinstance(b, str):
        return a.strip() == b.strip()
    if isinstance(a, num) and isinstance(b, num):
        return float(a) == float(b)
    if isinstance(a, str) and isinstance(b, num) or isinstance(a, num) and isinstance(b, str):
        s, x = (a, b) if isinstance(a, str) else (b, a)
        try:
            return float(s.strip()) == float(x)
        except ValueError:
            return False
    return a == b


def calls_match(exp_name: str, exp_args: Dict, got: Optional[Dict]) -> bool:
    if not got or got.get("name") != exp_name:
        return False
    g = got.get("arguments")
    if not isinstance(g, dict) or len(g) != len(exp_args):
        return g == exp_args
    return all(k in g and _val_eq(v, g[k]) for k, v in exp_args.items())


def first_tool_call(text: str) -> Optional[Dict]:
    calls, _ = parse_tool_calls(text)
    return calls[0] if calls else None
