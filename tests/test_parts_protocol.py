"""Optional abilities of parts are declared, and a declaration that does not match the part is an
error when the block is built, not a fusion that is silently lost."""
import pytest
import torch

from firefly_b200.config.base import ConfigError, LayerSpec, PartSpec
from firefly_b200.parts import Runtime, register_part
from firefly_b200.parts.base import Part, declared
from firefly_b200.parts.block import PreNormBlock


class _MisspeltKeyword(Part):
    adds_into_residual = True

    def __init__(self, spec, rt, position=None):
        super().__init__(spec, rt)

    def cache_spec(self):
        return None

    def forward(self, x, ctx, slot, write_cache, accumulate_in=None):
        return x


class _UndeclaredKeyword(Part):
    def forward(self, x, ctx, accumulate_into=None):
        return x


class _FoldsWithoutAdding(Part):
    folds_next_norm = True

    def forward(self, x, ctx, then_norm=None):
        return x


class _NotAPart:                      # parts need not derive from Part
    def forward(self, x, ctx):
        return x


def test_declarations_are_checked_both_ways():
    sp = PartSpec("k", {})
    with pytest.raises(ConfigError, match="no 'accumulate_into' keyword"):
        declared(_MisspeltKeyword(sp, None), "adds_into_residual")
    with pytest.raises(ConfigError, match="does not declare adds_into_residual"):
        declared(_UndeclaredKeyword(sp, None), "adds_into_residual")
    with pytest.raises(ConfigError, match="without adds_into_residual"):
        declared(_FoldsWithoutAdding(sp, None), "folds_next_norm")
    assert declared(_NotAPart(), "adds_into_residual") is False
    assert declared(_NotAPart(), "foldable") is False


def test_a_block_with_a_misdeclared_part_is_refused_when_it_is_built():
    register_part("mixer", "misspelt_keyword_mixer", _MisspeltKeyword, replace=True)
    norm = PartSpec("rms_norm", dict(size=8, eps=1e-6), prefix="n")
    layer = LayerSpec(arrangement="pre_norm", mixer=PartSpec("misspelt_keyword_mixer", {}, prefix="m"),
                      feed_forward=PartSpec("swiglu_mlp", dict(hidden_size=8, intermediate_size=16), prefix="f"),
                      norms=(norm, norm), position=None)
    with pytest.raises(ConfigError, match="_MisspeltKeyword declares adds_into_residual"):
        PreNormBlock(layer, Runtime(torch.device("cpu"), torch.float32))


def test_the_engines_own_parts_declare_what_they_do():
    from firefly_b200.parts.attention import GQAttention
    from firefly_b200.parts.mlp import SwiGLUMLP
    from firefly_b200.parts.norm import RMSNorm
    for cls in (GQAttention, SwiGLUMLP):
        assert cls.adds_into_residual and cls.folds_next_norm and cls.accepts_folded_norm
    assert RMSNorm.foldable and PreNormBlock.takes_next_norm


def test_a_part_that_synchronises_with_the_host_is_found_through_the_parts_that_hold_it():
    from firefly_b200.parts.base import host_synchronous

    class Quiet:
        pass

    class Loud:
        host_synchronous = True

    class Holder:
        def __init__(self, inner):
            self.inner = inner

        def parts(self):
            return self.inner

    assert not host_synchronous(Quiet())
    assert host_synchronous(Loud())
    assert not host_synchronous(Holder([Quiet(), Holder([Quiet()])]))
    assert host_synchronous(Holder([Quiet(), Holder([Loud()])]))
    # the package's own model has none, so its steps may be captured
    import plain_qwen3 as P
    from firefly_b200.models import DecoderModel, config_from_dict, spec_for
    model = DecoderModel(spec_for(config_from_dict(P.TINY_A)), Runtime(torch.device("cpu"), torch.float32))
    assert model.host_synchronous is False
    assert len(model.blocks[0].parts()) >= 4
