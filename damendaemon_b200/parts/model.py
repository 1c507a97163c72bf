"""A decoder assembled from parts according to a ModelSpec. Architecture-agnostic."""
from __future__ import annotations

import torch

from .. import kernels
from . import (attention, block, delta_rule, embedding, feed_forward, head, latent_attention, linear_recurrence, norms,  # noqa: F401
               positions, retention, side_by_side, state_space)  # noqa: F401  (register the built-in parts)
from .spec import TensorDecl
from .registry import ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, lookup


def tensor_decls(spec):
    """Every checkpoint tensor the model wants, each name once."""
    decls = list(lookup(EMBEDDINGS, spec.embedding, "embedding").tensor_decls(spec.embedding))
    decls += lookup(POSITIONS, spec.position, "position encoding").tensor_decls(spec.position)
    for layer in spec.layers:
        for norm in layer.norms:
            decls += lookup(NORMS, norm, "norm").tensor_decls(norm)
        decls += lookup(MIXERS, layer.mixer, "mixer").tensor_decls(layer.mixer)
        decls += lookup(FEED_FORWARDS, layer.feed_forward, "feed-forward").tensor_decls(layer.feed_forward)
        decls += getattr(lookup(ARRANGEMENTS, layer, "block arrangement"), "tensor_decls", lambda _: [])(layer)
    decls += lookup(HEADS, spec.head, "head").tensor_decls(spec.head)
    for stop, name in enumerate(spec.depth_mix or ()):
        decls.append(TensorDecl(name, (stop + 2,), "vector"))
    if spec.pass_vectors is not None:
        decls.append(TensorDecl(spec.pass_vectors[0], (spec.pass_vectors[1], spec.width), "vector"))
    unique = {}
    for d in decls:
        if d.name in unique and unique[d.name] != d:
            raise ValueError(f"tensor {d.name} is declared twice with different shapes or roles")
        unique[d.name] = d
    return list(unique.values())


def cache_needs(spec):
    """One list of cache needs per stop of the run order: the mixer's (none for a stop that reads another's cache) and
    the block arrangement's own (a state with a name); then, where the embedding has needs of its own, one more list with them."""
    needs = []
    for entry in spec.run_order:
        layer = spec.layers[entry.layer]
        mixer = layer.mixer
        mine = [] if entry.cache_of is not None else list(lookup(MIXERS, mixer, "mixer").cache_needs(mixer))
        mine += getattr(lookup(ARRANGEMENTS, layer, "block arrangement"), "cache_needs", lambda _: [])(layer)
        needs.append(mine)
    # one more site after the stops: the embedding's own per-request state, if it has any
    own = list(getattr(lookup(EMBEDDINGS, spec.embedding, "embedding"), "cache_needs", lambda _: [])(spec.embedding))
    if own:
        needs.append(own)
    return needs


class DecoderModel:
    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        for stop, entry in enumerate(spec.run_order):
            if not 0 <= entry.layer < len(spec.layers):
                raise ValueError(f"stop {stop} of the run order names layer {entry.layer}; the model has {len(spec.layers)}")
            if entry.cache_of is not None and (not 0 <= entry.cache_of < stop or
                                               spec.run_order[entry.cache_of].cache_of is not None):
                raise ValueError(f"stop {stop} reads the cache of stop {entry.cache_of}, which must be an earlier stop "
                                 "with a cache of its own")
        self.embedding = lookup(EMBEDDINGS, spec.embedding, "embedding")(spec.embedding, weights, runtime)
        self.position = lookup(POSITIONS, spec.position, "position encoding")(spec.position, weights, runtime)
        self.blocks, self.mixers, self.feed_forwards = [], [], []
        for layer in spec.layers:
            mixer = lookup(MIXERS, layer.mixer, "mixer")(layer.mixer, weights, runtime)
            feed = lookup(FEED_FORWARDS, layer.feed_forward, "feed-forward")(layer.feed_forward, weights, runtime)
            built_norms = [lookup(NORMS, norm, "norm")(norm, weights, runtime) for norm in layer.norms]
            self.blocks.append(lookup(ARRANGEMENTS, layer, "block arrangement")(layer, built_norms, mixer, feed))
            if hasattr(self.blocks[-1], "bind"):
                self.blocks[-1].bind(weights)           # an arrangement with tensors of its own
            self.mixers.append(mixer)
            self.feed_forwards.append(feed)
        self.head = lookup(HEADS, spec.head, "head")(spec.head, weights, runtime)
        self.depth_mix = None
        if spec.depth_mix is not None:
            if len(spec.depth_mix) != len(spec.run_order):
                raise ValueError(f"{len(spec.depth_mix)} depth weights for {len(spec.run_order)} stops of the run order")
            self.depth_mix = [weights[name] for name in spec.depth_mix]
        self.pass_vectors = None
        if spec.pass_vectors is not None:
            self.pass_vectors = weights[spec.pass_vectors[0]]
        for stop, entry in enumerate(spec.run_order):
            if entry.add_vector is not None and (self.pass_vectors is None or not 0 <= entry.add_vector < self.pass_vectors.shape[0]):
                raise ValueError(f"stop {stop} adds row {entry.add_vector} of a table the model does not have")
        if spec.depth_mix is not None and any(e.add_embedding or e.add_vector is not None for e in spec.run_order):
            raise ValueError("streams mixed over depth and stops that add to the stream do not go together")
        self.keeps_embedding = any(e.add_embedding for e in spec.run_order)
        self.embedding_has_state = bool(getattr(self.embedding, "cache_needs", lambda _: [])(spec.embedding))
        self.graph_safe = all(getattr(m, "graph_safe", False) for m in self.mixers) and \
            all(getattr(f, "graph_safe", False) for f in self.feed_forwards)
        # where the mixers like a prompt to be cut (a key block of a prompt attention kernel); 1: anywhere
        self.portion_multiple = max([int(getattr(m, "portion_multiple", 1)) for m in self.mixers] + [1])

    def forward(self, ctx, caches):
        """Run the step's tokens; float32 logits [wanted rows, vocab] (or None if none are wanted).

        caches: per stop of the run order, the LayerCache view its mixer reads (and writes, if it is its own); after
        them the view of the embedding's own site.
        """
        if self.embedding_has_state:
            x = self.embedding.forward(ctx, self.position, caches[len(self.spec.run_order)])
        else:
            x = self.embedding.forward(ctx, self.position)
        if self.depth_mix is not None:
            x = self._forward_mixed_over_depth(x, ctx, caches)
        else:
            first = x.clone() if self.keeps_embedding else None       # the blocks write the stream in place
            for stop, entry in enumerate(self.spec.run_order):
                if entry.add_embedding or entry.add_vector is not None:
                    kernels.add_rows(x, first if entry.add_embedding else None,
                                     None if entry.add_vector is None else self.pass_vectors[entry.add_vector])
                x = self.blocks[entry.layer].forward(x, ctx, caches[stop], self.position)
        if ctx.n_wanted == 0:
            return None
        return self.head.forward(x, ctx)

    def _forward_mixed_over_depth(self, x, ctx, caches):
        """Every stop's result stays: plane 0 of the stack is the embedding's output, plane i + 1 what stop i leaves. A stop
        runs in place on the plane that will hold its result, which first receives what the stop reads: a copy of plane 0 for
        the first stop, else the weighted sum of all planes so far by the weights of the stop before."""
        stops = len(self.spec.run_order)
        stack = torch.empty((stops + 2, *x.shape), dtype=torch.float32, device=x.device)
        stack[0].copy_(x)
        stack[1].copy_(x)
        for stop, entry in enumerate(self.spec.run_order):
            self.blocks[entry.layer].forward(stack[stop + 1], ctx, caches[stop], self.position)
            kernels.weighted_sum(stack, self.depth_mix[stop], stop + 2, stack[stop + 2])
        return stack[stops + 1]
