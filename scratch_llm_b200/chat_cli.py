"""Command line in the manner of the reference's ``python -m scratch_llm.chat_cli``
(src/scratch_llm/chat_cli.py:125-156): a read-eval-print loop that renders the conversation
with the chat template, generates greedily until ``<|eot|>`` or ``--max-tokens``, and prints
the reply.

    python -m scratch_llm_b200.chat_cli --model DIR [--data-dir DIR] [--max-tokens 256]
        [--temperature 0.0] [--top-p 1.0] [--seed N] [--dtype bfloat16|float32]
        [--random-weights CONFIG.json]

``--model`` takes the place of the reference's ``--ckpt`` (a model folder instead of a pickle;
``--ckpt`` is accepted as another spelling); ``--data-dir`` is the folder with
``tokenizer.json`` as in the reference (default: the model folder) and ``--max-tokens`` keeps
its meaning and default; ``--device`` is accepted but can only be ``cuda``.  Without a tokenizer (a random-weights folder) the
loop reads and prints token ids.  ``--random-weights CONFIG.json`` first writes ``--model`` from
that configuration with seeded random weights.

Template (src/scratch_llm/chat.py:30-115): ``<|bos|>`` then per turn ``<|user|>`` or
``<|assistant|>``, the content, ``<|eot|>``; the prompt for a reply ends with ``<|assistant|>``.
"""

from __future__ import annotations

import argparse
import json
import sys
from dataclasses import dataclass, field
from pathlib import Path

BOS, USER, ASSISTANT, EOT = "<|bos|>", "<|user|>", "<|assistant|>", "<|eot|>"
SPECIALS = [BOS, USER, ASSISTANT, EOT]


def special_id(tokenizer, token: str) -> int:
    ids = tokenizer.encode(token)
    if len(ids) != 1:
        raise ValueError(f"special token {token!r} encodes to {len(ids)} ids, expected 1: this "
                         "tokenizer was not made with the chat special tokens")
    return ids[0]


def render_for_completion(messages: list[tuple[str, str]], tokenizer) -> list[int]:
    ids = [special_id(tokenizer, BOS)]
    for role, content in messages:
        if role not in ("user", "assistant"):
            raise ValueError(f"unknown role {role!r}")
        ids.append(special_id(tokenizer, USER if role == "user" else ASSISTANT))
        ids.extend(tokenizer.encode(content))
        ids.append(special_id(tokenizer, EOT))
    ids.append(special_id(tokenizer, ASSISTANT))
    return ids


@dataclass
class ChatSession:
    """Multi-turn chat (src/scratch_llm/chat_cli.py:57-100 of the reference): every reply
    renders the whole history again and decodes it from an empty cache."""

    llm: object
    tokenizer: object
    max_tokens: int = 256
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int | None = None
    history: list[tuple[str, str]] = field(default_factory=list)

    def reply(self, user_text: str) -> str:
        from .sampling import SamplingParams

        eot = special_id(self.tokenizer, EOT)
        specials = {special_id(self.tokenizer, s) for s in SPECIALS}
        prompt = render_for_completion([*self.history, ("user", user_text)], self.tokenizer)
        gen = self.llm.generate(prompt, SamplingParams(
            temperature=self.temperature, top_p=self.top_p, max_tokens=self.max_tokens,
            stop_ids=(eot,), seed=self.seed))
        answer = []
        for t in gen:
            if t == eot:
                break
            if t not in specials:
                answer.append(t)
        text = self.tokenizer.decode(answer)
        self.history += [("user", user_text), ("assistant", text)]
        return text

    def reset(self) -> None:
        self.history.clear()


def batch_reply(llm, tokenizer, user_texts, *, max_tokens: int = 256) -> list[str]:
    """Greedy replies to independent single-turn messages, as one continuous batch
    (src/scratch_llm/chat_cli.py:103-122 of the reference, without its equal-length limit)."""
    from .sampling import SamplingParams

    eot = special_id(tokenizer, EOT)
    specials = {special_id(tokenizer, s) for s in SPECIALS}
    prompts = [render_for_completion([("user", t)], tokenizer) for t in user_texts]
    gens = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=max_tokens,
                                                stop_ids=(eot,)))
    out = []
    for g in gens:
        cut = g[:g.index(eot)] if eot in g else g
        out.append(tokenizer.decode([t for t in cut if t not in specials]))
    return out


def repl(llm, tokenizer, args) -> None:
    from .sampling import SamplingParams

    print("chat - Ctrl-D to exit" if tokenizer else
          "no tokenizer.json: type token ids separated by spaces - Ctrl-D to exit")
    session = ChatSession(llm, tokenizer, args.max_tokens, args.temperature, args.top_p,
                          args.seed) if tokenizer else None
    while True:
        try:
            line = input("you> ")
        except EOFError:
            print()
            return
        if session:
            print("bot>", session.reply(line))
            continue
        try:
            ids = [int(t) for t in line.replace(",", " ").split()]
        except ValueError:
            print("bot> (token ids are integers)")
            continue
        if not ids:
            continue
        gen = llm.generate(ids, SamplingParams(temperature=args.temperature, top_p=args.top_p,
                                               max_tokens=args.max_tokens, seed=args.seed))
        print("bot>", " ".join(map(str, gen)))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Chat with a model folder on one B200.")
    ap.add_argument("--model", "--ckpt", dest="model", required=True,
                    help="folder with config.json and model.safetensors (--ckpt, the reference's "
                         "name for its checkpoint option, is accepted too)")
    ap.add_argument("--device", default="cuda",
                    help="kept from the reference's command line; only 'cuda' is possible")
    ap.add_argument("--data-dir", default=None, help="dir with tokenizer.json (default: --model)")
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--random-weights", metavar="CONFIG.json", default=None,
                    help="write --model from this configuration with seeded random weights first")
    args = ap.parse_args(argv)
    if not str(args.device).startswith("cuda"):
        ap.error("this engine runs on a CUDA device only (--device cuda)")

    if args.random_weights:
        from .config import config_from_dict
        from .weights import write_random_model
        cfg = config_from_dict(json.loads(Path(args.random_weights).read_text()))
        write_random_model(cfg, args.model, args.seed or 0)
    from .engine import LLM
    from .tokenizer import Tokenizer

    tok_path = Path(args.data_dir or args.model) / "tokenizer.json"
    tokenizer = Tokenizer.load(tok_path) if tok_path.is_file() else None
    llm = LLM(args.model, dtype=args.dtype, verbose=True)
    repl(llm, tokenizer, args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
