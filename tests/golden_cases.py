"""Seeded, integer-generated inputs shared by the golden-fixture generator and the tests that replay them."""
import numpy as np

import fixtures


def small_layer(type_: int, channels: int = 256, hidden: int = 256, experts: int = 6, selected: int = 3, tokens: int = 5):
    """A whole MoE layer with bounded-domain weights (every |w| <= 1/256) and LCG activations."""
    seeds = iter(range(101, 120))
    g = fixtures.bounded_weights(type_, channels, hidden, experts, next(seeds))
    u = fixtures.bounded_weights(type_, channels, hidden, experts, next(seeds))
    d = fixtures.bounded_weights(type_, hidden, channels, experts, next(seeds))
    sg = fixtures.bounded_weights(type_, channels, hidden, 1, next(seeds))[0]
    su = fixtures.bounded_weights(type_, channels, hidden, 1, next(seeds))[0]
    sd = fixtures.bounded_weights(type_, hidden, channels, 1, next(seeds))[0]
    sr = fixtures.lcg_activations(next(seeds), channels) * np.float32(0.125)
    layer = dict(channels=channels, hidden=hidden, experts=experts, selected=selected, expert_type=type_, shared_type=type_,
                 gate=g, up=u, down=d, shared_gate=sg, shared_up=su, shared_down=sd, shared_router=sr, router=None,
                 mode=0, normalize=True)
    x = fixtures.lcg_activations(next(seeds), tokens * channels).reshape(tokens, channels) * np.float32(16)
    logits = fixtures.lcg_activations(next(seeds), tokens * experts).reshape(tokens, experts) * np.float32(3)
    logits[1, :] = np.float32(0.5)       # a row of exact ties: ids must come out 0,1,2
    logits[2, 4] = logits[2, 1]          # one pairwise tie
    return layer, x.astype(np.float32), logits.astype(np.float32)
