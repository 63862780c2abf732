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


def five_bit_layer(channels: int = 256, hidden: int = 64, experts: int = 4, selected: int = 2, tokens: int = 4):
    """The reference model's other pairing (model.cpp:52-57): Q5_K gate / up, Q5_1 down, Q8_0 shared expert. Expert bytes come
    straight from the LCG (every code and factor pattern), with small binary16 scales so that the sums stay moderate."""
    def lcg(type_, cols, rows, n, seed):
        w = fixtures.lcg_weights(type_, cols, rows, n, seed=seed).copy()
        bpb = fixtures.block_bytes(type_)
        blocks = w.reshape(n, -1, bpb)
        blocks[:, :, 0] = 1; blocks[:, :, 1] = 0x0c            # d = 0x0c01
        blocks[:, :, 2] = 1; blocks[:, :, 3] = 0x04            # dmin (Q5_K) / m (Q5_1) = 0x0401
        return w
    g, u = lcg(13, channels, hidden, experts, 201), lcg(13, channels, hidden, experts, 202)
    d = lcg(7, hidden, channels, experts, 203)
    sg = fixtures.bounded_weights(8, channels, hidden, 1, 204)[0]
    su = fixtures.bounded_weights(8, channels, hidden, 1, 205)[0]
    sd = fixtures.bounded_weights(8, hidden, channels, 1, 206)[0]
    sr = fixtures.lcg_activations(207, channels) * np.float32(0.125)
    layer = dict(channels=channels, hidden=hidden, experts=experts, selected=selected, expert_type=13, shared_type=8, down_type=7,
                 gate=g, up=u, down=d, shared_gate=sg, shared_up=su, shared_down=sd, shared_router=sr, router=None,
                 mode=0, normalize=True)
    x = fixtures.lcg_activations(208, tokens * channels).reshape(tokens, channels) * np.float32(4)
    logits = fixtures.lcg_activations(209, tokens * experts).reshape(tokens, experts) * np.float32(3)
    return layer, x.astype(np.float32), logits.astype(np.float32)
