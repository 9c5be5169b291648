"""``hmf chat CKPT``: interactive terminal chat on the native engine."""
from __future__ import annotations

import argparse

import torch

from ..data.formats import get_template, load_tokenizer
from ..utils import checkpoint_io
from .engine import SamplingParams, ServingEngine


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="hmf chat")
    ap.add_argument("model")
    ap.add_argument("--template", default=None)
    ap.add_argument("--max-new-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.0)
    args = ap.parse_args(argv)
    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    model = checkpoint_io.from_pretrained(args.model, device=device, init="meta")
    tok, tpl = load_tokenizer(args.model), get_template(args.template)
    engine = ServingEngine(model, max_num_seqs=1, max_model_len=8192)
    history = []
    print("type `exit` to quit, `clear` to reset the conversation")
    while True:
        try:
            text = input("User: ")
        except EOFError:
            break
        if text.strip() == "exit":
            break
        if text.strip() == "clear":
            history = []
            continue
        history.append({"role": "user", "content": text})
        pairs = tpl.encode_multiturn(tok, history + [{"role": "assistant", "content": ""}])
        ids = []
        for i, (p, r) in enumerate(pairs):
            ids += p + (r if i < len(pairs) - 1 else [])
        out = engine.generate([ids], SamplingParams(max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                                                     eos_token_id=getattr(tok, "eos_token_id", None), ignore_eos=False))[0]
        reply = tok.decode(out)
        print("Assistant:", reply)
        history.append({"role": "assistant", "content": reply})
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
