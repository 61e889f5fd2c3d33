"""Holding greedily generated tokens to the plain implementation, near-ties included."""
import torch

import plain_llama


def check_greedy(cfg, w, prompt, tokens, margin, what=""):
    """Every token of ``tokens`` (generated greedily after ``prompt``) against the plain
    implementation run on the same tokens before it.  Where the plain top-two margin is at least
    ``margin`` the token has to be the plain arg-max; where the two are closer than the rounding
    of the engine's dtype, the token has to be one of those within ``margin`` of the top (either
    is a right answer there, and the sequence goes on from the engine's choice).  Returns how
    many tokens were of the first kind."""
    toks, strict = list(prompt), 0
    for k, t in enumerate(tokens):
        logits = plain_llama.forward_logits(cfg, w, toks)[-1]
        top = torch.topk(logits, 2).values
        if float(top[0] - top[1]) >= margin:
            assert t == int(torch.argmax(logits)), \
                f"{what}: token {k} is {t}, plain says {int(torch.argmax(logits))} by {float(top[0] - top[1]):.3g}"
            strict += 1
        else:
            assert float(top[0] - logits[t]) < margin, \
                f"{what}: token {k} is {t}, {float(top[0] - logits[t]):.3g} below the plain top"
        toks.append(t)
    return strict
