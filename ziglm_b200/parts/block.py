"""The pre-norm residual arrangement: x += mixer(norm(x)); x += ffn(norm(x)).

This is the reference's layer body for the architectures without post-norms:
norm, attention, residual sum, norm, feed-forward, residual sum
(src/model.zig:545-546,704-716,719-755).  The residual stream x is float32 in
both precisions; mixers and feed-forwards add into it themselves, so the sum
rides in the epilogue of their last matrix product.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import LayerSpec
from .base import (KVNeed, LayerIO, ParamDecl, Part, StateNeed, feed_forward_class, mixer_class, norm_class,
                   register_block)


class PreNormBlock(Part):
    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        self.mixer_norm = norm_class(spec.mixer_norm.kind)(spec.mixer_norm, dtype, device)
        self.mixer = mixer_class(spec.mixer.kind)(spec.mixer, dtype, device)
        self.ffn_norm = norm_class(spec.ffn_norm.kind)(spec.ffn_norm, dtype, device)
        self.ffn = feed_forward_class(spec.ffn.kind)(spec.ffn, dtype, device)

    @classmethod
    def _children(cls, spec: LayerSpec):
        return (("mixer_norm.", norm_class(spec.mixer_norm.kind), spec.mixer_norm),
                ("mixer.", mixer_class(spec.mixer.kind), spec.mixer),
                ("ffn_norm.", norm_class(spec.ffn_norm.kind), spec.ffn_norm),
                ("ffn.", feed_forward_class(spec.ffn.kind), spec.ffn))

    @classmethod
    def declare(cls, spec: LayerSpec) -> Dict[str, ParamDecl]:
        out: Dict[str, ParamDecl] = {}
        for prefix, klass, sub in cls._children(spec):
            for name, decl in klass.declare(sub).items():
                out[prefix + name] = decl
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in (("mixer_norm.", self.mixer_norm), ("mixer.", self.mixer),
                             ("ffn_norm.", self.ffn_norm), ("ffn.", self.ffn)):
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def kernel_libraries(self) -> Tuple[str, ...]:
        return (self.mixer_norm.kernel_libraries() + self.mixer.kernel_libraries()
                + self.ffn_norm.kernel_libraries() + self.ffn.kernel_libraries())

    def cache_needs(self) -> Optional[KVNeed]:
        return self.mixer.cache_needs()

    def state_needs(self) -> Optional[StateNeed]:
        return self.mixer.state_needs()

    def accepts_normed_input(self) -> bool:
        """Whether ``forward`` may be handed this block's first norm half done (``h_in``)."""
        return bool(self.mixer_norm.fusable and self.mixer.takes_normed_input)

    def forward(self, step, io: LayerIO, x: torch.Tensor, h_in=None, next_norm=None):
        """``h_in``: this block's first norm, half done by the block before (else the norm kernel runs).
        ``next_norm``: the first norm of the block after; the result is its half-done form if the feed-forward's
        last product did it, else None."""
        h = h_in if h_in is not None else self.mixer_norm.forward(step, x)
        if self.mixer.fuses_next_norm and self.ffn.takes_normed_input and self.ffn_norm.fusable:
            h = self.mixer.forward(step, io, h, x, next_norm=self.ffn_norm)
        else:
            self.mixer.forward(step, io, h, x)
            h = None
        if h is None:
            h = self.ffn_norm.forward(step, x)
        if self.ffn.fuses_next_norm and next_norm is not None:
            return self.ffn.forward(step, h, x, next_norm=next_norm)
        self.ffn.forward(step, h, x)
        return None


register_block("prenorm", PreNormBlock)


class SandwichBlock(Part):
    """Norms before and after each sublayer: x += post1(mixer(pre1(x))); x += post2(ffn(pre2(x))).

    The two post-norms come in ``LayerSpec.options`` (``mixer_post_norm``, ``ffn_post_norm``); a layer whose spec
    has no feed-forward (``ffn`` and ``ffn_norm`` are None) ends after the mixer.  A sublayer writes its output
    into a float32 branch buffer of the step's scratch (a part that sets ``can_overwrite`` is asked to overwrite
    it, for any other the buffer is zeroed first and the part adds into it, as it would into the residual); the
    post-norm then reads the branch in float32 and adds the normed rows into the residual in the same kernel,
    which also leaves the rows of the norm before the next sublayer (of this block or of the next one).
    """

    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        self.parts: Dict[str, Part] = {}
        for prefix, klass, sub in self._children(spec):
            self.parts[prefix] = klass(sub, dtype, device)
        self.mixer_norm = self.parts["mixer_norm."]
        self.mixer = self.parts["mixer."]
        self.mixer_post = self.parts["mixer_post_norm."]
        self.ffn_norm = self.parts.get("ffn_norm.")
        self.ffn = self.parts.get("ffn.")
        self.ffn_post = self.parts.get("ffn_post_norm.")

    @classmethod
    def _children(cls, spec: LayerSpec):
        post = spec.options["mixer_post_norm"]
        out = [("mixer_norm.", norm_class(spec.mixer_norm.kind), spec.mixer_norm),
               ("mixer.", mixer_class(spec.mixer.kind), spec.mixer),
               ("mixer_post_norm.", norm_class(post.kind), post)]
        if spec.ffn is not None:
            post = spec.options["ffn_post_norm"]
            out += [("ffn_norm.", norm_class(spec.ffn_norm.kind), spec.ffn_norm),
                    ("ffn.", feed_forward_class(spec.ffn.kind), spec.ffn),
                    ("ffn_post_norm.", norm_class(post.kind), post)]
        return out

    @classmethod
    def declare(cls, spec: LayerSpec) -> Dict[str, ParamDecl]:
        out: Dict[str, ParamDecl] = {}
        for prefix, klass, sub in cls._children(spec):
            for name, decl in klass.declare(sub).items():
                out[prefix + name] = decl
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in self.parts.items():
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs: Tuple[str, ...] = ()
        for part in self.parts.values():
            libs += part.kernel_libraries()
        return libs

    def cache_needs(self) -> Optional[KVNeed]:
        return self.mixer.cache_needs()

    def state_needs(self) -> Optional[StateNeed]:
        return self.mixer.state_needs()

    def accepts_normed_input(self) -> bool:
        """The block before may hand this block's first norm over as finished rows (``h_in``)."""
        return bool(self.mixer_norm.fusable)

    @staticmethod
    def _branch(step, part, x: torch.Tensor) -> torch.Tensor:
        branch = step.ws.buf("branch", tuple(x.shape), torch.float32)
        if not part.can_overwrite:
            branch.zero_()
        return branch

    def _close(self, step, post, branch: torch.Tensor, x: torch.Tensor, nxt, name: str):
        """x += post(branch); with ``nxt`` (the norm of the sublayer that follows, here or in the next block) also
        its rows of the new x, from the same kernel.  Returns those rows or None."""
        if nxt is not None and hasattr(post, "add_normed_then") and getattr(nxt, "fusable", False):
            return post.add_normed_then(step, branch, x, nxt, name=name)
        post.add_normed(step, branch, x)
        return None

    def forward(self, step, io: LayerIO, x: torch.Tensor, h_in=None, next_norm=None):
        """``h_in``: this block's first norm, done by the block before (finished rows; a half-done norm of the
        kind the products of a pre-norm block carry is not taken).  ``next_norm``: the first norm of the block
        after; the result is its rows if this block's last kernel made them, else None."""
        h = h_in if isinstance(h_in, torch.Tensor) else self.mixer_norm.forward(step, x)
        branch = self._branch(step, self.mixer, x)
        if self.mixer.can_overwrite:
            self.mixer.forward(step, io, h, branch, accumulate=False)
        else:
            self.mixer.forward(step, io, h, branch)
        if self.ffn is None:
            return self._close(step, self.mixer_post, branch, x, next_norm, "norm_out_next")
        h = self._close(step, self.mixer_post, branch, x, self.ffn_norm, "norm_out_ffn")
        if h is None:
            h = self.ffn_norm.forward(step, x)
        branch = self._branch(step, self.ffn, x)
        if self.ffn.can_overwrite:
            self.ffn.forward(step, h, branch, accumulate=False)
        else:
            self.ffn.forward(step, h, branch)
        return self._close(step, self.ffn_post, branch, x, next_norm, "norm_out_next")


register_block("sandwich", SandwichBlock)


class PostNormBlock(Part):
    """Norms behind the sublayers only, and a multiplier on what they add: x += m * post1(mixer(x)) and, where the
    layer has a feed-forward, x += m * post2(ffn(x)).  The sublayers read the residual stream itself (its rows in
    the step's storage type; in float32 the residual as it is).

    The two post-norms come in ``LayerSpec.options`` (``mixer_post_norm``, ``ffn_post_norm``) and m as
    ``residual_mult`` (default 1).  A sublayer writes its output into a float32 branch buffer; the post-norm reads
    it in float32, adds the multiplied rows into the residual and leaves the new rows for the sublayer that follows,
    here or in the next block, all in one kernel.  ``mixer_norm`` is the part that makes those rows when nobody has
    (the first block of a model, or a block behind one of another arrangement)."""

    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        self.mult = float(spec.options.get("residual_mult", 1.0))
        self.mixer_norm = norm_class("cast")(None, dtype, device)
        self.parts: Dict[str, Part] = {}
        for prefix, klass, sub in self._children(spec):
            self.parts[prefix] = klass(sub, dtype, device)
        self.mixer = self.parts["mixer."]
        self.mixer_post = self.parts["mixer_post_norm."]
        self.ffn = self.parts.get("ffn.")
        self.ffn_post = self.parts.get("ffn_post_norm.")

    @classmethod
    def _children(cls, spec: LayerSpec):
        post = spec.options["mixer_post_norm"]
        out = [("mixer.", mixer_class(spec.mixer.kind), spec.mixer),
               ("mixer_post_norm.", norm_class(post.kind), post)]
        if spec.ffn is not None:
            post = spec.options["ffn_post_norm"]
            out += [("ffn.", feed_forward_class(spec.ffn.kind), spec.ffn),
                    ("ffn_post_norm.", norm_class(post.kind), post)]
        return out

    @classmethod
    def declare(cls, spec: LayerSpec) -> Dict[str, ParamDecl]:
        out: Dict[str, ParamDecl] = {}
        for prefix, klass, sub in cls._children(spec):
            for name, decl in klass.declare(sub).items():
                out[prefix + name] = decl
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in self.parts.items():
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs: Tuple[str, ...] = self.mixer_norm.kernel_libraries()
        for part in self.parts.values():
            libs += part.kernel_libraries()
        return libs

    def cache_needs(self) -> Optional[KVNeed]:
        return self.mixer.cache_needs()

    def state_needs(self) -> Optional[StateNeed]:
        return self.mixer.state_needs()

    def accepts_normed_input(self) -> bool:
        """The block before may hand over the rows this block's mixer reads (``h_in``)."""
        return True

    def _close(self, step, post, branch: torch.Tensor, x: torch.Tensor, want_rows: bool, name: str):
        """x += m * post(branch); with ``want_rows`` also the new rows of x for the sublayer that follows."""
        if hasattr(post, "add_scaled"):
            if not want_rows or self.dtype == torch.float32:
                post.add_scaled(step, branch, x, self.mult)
                return x if want_rows else None
            return post.add_scaled(step, branch, x, self.mult, rows_out=step.ws.buf(name, tuple(x.shape), self.dtype))
        # a norm without the fused form: norm into the branch's own rows, multiply, add
        normed = step.ws.buf("branch_normed", tuple(x.shape), torch.float32)
        post.forward_rows(branch, normed)
        if self.mult != 1.0:
            kernels.scale_(normed, self.mult)
        kernels.add_(x, normed)
        return self.mixer_norm.forward(step, x, name=name) if want_rows else None

    def forward(self, step, io: LayerIO, x: torch.Tensor, h_in=None, next_norm=None):
        """``h_in``: the rows the mixer reads, left by the block before.  ``next_norm``: the first part of the block
        after; if that block reads the residual itself (its part is the cast) the result is the rows it reads."""
        h = h_in if isinstance(h_in, torch.Tensor) else self.mixer_norm.forward(step, x, name="rows_mixer")
        feeds_next = type(next_norm) is type(self.mixer_norm)
        branch = step.ws.buf("branch", tuple(x.shape), torch.float32)
        if self.mixer.can_overwrite:
            self.mixer.forward(step, io, h, branch, accumulate=False)
        else:
            branch.zero_()
            self.mixer.forward(step, io, h, branch)
        if self.ffn is None:
            return self._close(step, self.mixer_post, branch, x, feeds_next, "rows_next")
        h = self._close(step, self.mixer_post, branch, x, True, "rows_ffn")
        branch = step.ws.buf("branch", tuple(x.shape), torch.float32)
        if self.ffn.can_overwrite:
            self.ffn.forward(step, h, branch, accumulate=False)
        else:
            branch.zero_()
            self.ffn.forward(step, h, branch)
        return self._close(step, self.ffn_post, branch, x, feeds_next, "rows_next")


register_block("postnorm", PostNormBlock)


class SumNormBlock(Part):
    """Norms behind the sums: x <- post1(alpha x + mixer(x)) and, where the layer has a feed-forward,
    x <- post2(alpha x + ffn(x)).  The residual stream itself is normed after every sublayer, and the sublayers read it
    as it is (its rows in the step's storage type; in float32 the residual itself).

    The two norms come in ``LayerSpec.options`` (``mixer_post_norm``, ``ffn_post_norm``) and alpha as
    ``residual_mult`` (default 1).  A sublayer writes its output into a float32 branch buffer; the norm's kernel reads
    it, forms the sum and its norm in float32, writes the stream in place and leaves the new rows for the sublayer
    that follows, here or in the next block.  ``mixer_norm`` is the part that makes those rows when nobody has (the
    first block of a model, or a block behind one of another arrangement)."""

    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        self.alpha = float(spec.options.get("residual_mult", 1.0))
        self.mixer_norm = norm_class("cast")(None, dtype, device)
        self.parts: Dict[str, Part] = {}
        for prefix, klass, sub in self._children(spec):
            self.parts[prefix] = klass(sub, dtype, device)
        self.mixer = self.parts["mixer."]
        self.mixer_post = self.parts["mixer_post_norm."]
        self.ffn = self.parts.get("ffn.")
        self.ffn_post = self.parts.get("ffn_post_norm.")
        for post in (self.mixer_post, self.ffn_post):
            if post is not None and not hasattr(post, "sum_normed"):
                raise ValueError("sum_norm: the norm behind a sum must offer sum_normed")

    _children = PostNormBlock._children
    declare = PostNormBlock.declare
    bind = PostNormBlock.bind
    kernel_libraries = PostNormBlock.kernel_libraries
    cache_needs = PostNormBlock.cache_needs
    state_needs = PostNormBlock.state_needs

    def accepts_normed_input(self) -> bool:
        """The block before may hand over the rows this block's mixer reads (``h_in``)."""
        return True

    def _close(self, step, post, branch: torch.Tensor, x: torch.Tensor, want_rows: bool, name: str):
        """x <- post(alpha x + branch); with ``want_rows`` also the new rows of x for the sublayer that follows."""
        if not want_rows or self.dtype == torch.float32:
            post.sum_normed(step, branch, x, self.alpha)
            return x if want_rows else None
        return post.sum_normed(step, branch, x, self.alpha, rows_out=step.ws.buf(name, tuple(x.shape), self.dtype))

    def _run(self, part, step, io, h, x: torch.Tensor) -> torch.Tensor:
        branch = step.ws.buf("branch", tuple(x.shape), torch.float32)
        args = (step, h, branch) if io is None else (step, io, h, branch)
        if part.can_overwrite:
            part.forward(*args, accumulate=False)
        else:
            branch.zero_()
            part.forward(*args)
        return branch

    def forward(self, step, io: LayerIO, x: torch.Tensor, h_in=None, next_norm=None):
        """``h_in``: the rows the mixer reads, left by the block before.  ``next_norm``: the first part of the block
        after; if that block reads the residual itself (its part is the cast) the result is the rows it reads."""
        h = h_in if isinstance(h_in, torch.Tensor) else self.mixer_norm.forward(step, x, name="rows_mixer")
        feeds_next = type(next_norm) is type(self.mixer_norm)
        branch = self._run(self.mixer, step, io, h, x)
        if self.ffn is None:
            return self._close(step, self.mixer_post, branch, x, feeds_next, "rows_next")
        h = self._close(step, self.mixer_post, branch, x, True, "rows_ffn")
        branch = self._run(self.ffn, step, None, h, x)
        return self._close(step, self.ffn_post, branch, x, feeds_next, "rows_next")


register_block("sum_norm", SumNormBlock)


class SharedNormBlock(Part):
    """One norm whose rows the mixer and the feed-forward both read: with h = norm(x), x += mixer(h) + ff(h).

    The two sublayers add into the float32 residual one after the other; neither reads what the other wrote, so the
    sum is the arrangement's.  A layer whose spec has no feed-forward ends after the mixer.  ``spec.ffn_norm`` is not
    used (it is None)."""

    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        if spec.mixer_norm is None:
            raise ValueError("shared_norm: the arrangement needs the norm both sublayers read")
        self.parts: Dict[str, Part] = {}
        for prefix, klass, sub in self._children(spec):
            self.parts[prefix] = klass(sub, dtype, device)
        self.mixer_norm = self.parts["mixer_norm."]
        self.mixer = self.parts["mixer."]
        self.ffn = self.parts.get("ffn.")

    @classmethod
    def _children(cls, spec: LayerSpec):
        out = [("mixer_norm.", norm_class(spec.mixer_norm.kind), spec.mixer_norm),
               ("mixer.", mixer_class(spec.mixer.kind), spec.mixer)]
        if spec.ffn is not None:
            out.append(("ffn.", feed_forward_class(spec.ffn.kind), spec.ffn))
        return out

    @classmethod
    def declare(cls, spec: LayerSpec) -> Dict[str, ParamDecl]:
        out: Dict[str, ParamDecl] = {}
        for prefix, klass, sub in cls._children(spec):
            for name, decl in klass.declare(sub).items():
                out[prefix + name] = decl
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in self.parts.items():
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs: Tuple[str, ...] = ()
        for part in self.parts.values():
            libs += part.kernel_libraries()
        return libs

    def cache_needs(self) -> Optional[KVNeed]:
        return self.mixer.cache_needs()

    def state_needs(self) -> Optional[StateNeed]:
        return self.mixer.state_needs()

    def accepts_normed_input(self) -> bool:
        """The block before may hand this block's norm over as finished rows (``h_in``); a norm half done by a
        product is not taken, since two sublayers would have to complete it."""
        return False

    def forward(self, step, io: LayerIO, x: torch.Tensor, h_in=None, next_norm=None):
        h = h_in if isinstance(h_in, torch.Tensor) else self.mixer_norm.forward(step, x)
        self.mixer.forward(step, io, h, x)
        if self.ffn is not None:
            self.ffn.forward(step, h, x)
        return None


register_block("shared_norm", SharedNormBlock)
