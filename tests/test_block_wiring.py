"""How a block hands the next norm's work to its parts: only parts that say they can leave the norm's factor
to their successor are asked to, and only when the successor says it takes such rows (no GPU needed)."""
from aegean_tge_b200.parts.block import PreNormBlock


class _Norm:
    def __init__(self, log, name):
        self.log, self.name = log, name

    def forward(self, x, rows=None):
        self.log.append(("norm", self.name))
        return "normed"


class _Part:
    """Records the keyword arguments it is called with; an old-style part has no ``defer`` parameter at all."""

    def __init__(self, log, name, can_defer, takes_deferred, new_style=True):
        self.log, self.name = log, name
        self.can_defer_norm, self.takes_deferred_rows = can_defer, takes_deferred
        self.new_style = new_style

    def forward_add(self, h, x, ctx, *rest, next_norm=None, **more):
        if not self.new_style and more:
            raise TypeError(f"unexpected keyword arguments {sorted(more)}")
        self.log.append((self.name, h, more.get("defer", False)))
        return None if next_norm is None else f"rows of {self.name}"


def _block(log, mixer, feed_forward):
    return PreNormBlock(mixer, feed_forward, _Norm(log, "mixer_norm"), _Norm(log, "ffn_norm"), env=None)


def test_both_sides_must_agree_before_rows_travel_without_their_factor():
    for mixer_can, ffn_takes, ffn_can, next_takes in [(True, True, True, True), (True, False, True, True),
                                                      (False, True, True, False), (True, True, False, True)]:
        log = []
        mixer = _Part(log, "mixer", mixer_can, True)
        ffn = _Part(log, "ffn", ffn_can, ffn_takes)
        out = _block(log, mixer, ffn).forward("x", None, None, h=None, next_norm=_Norm(log, "next"),
                                              next_takes_deferred=next_takes)
        assert out == "rows of ffn"
        assert log[0] == ("norm", "mixer_norm")
        assert log[1] == ("mixer", "normed", mixer_can and ffn_takes)
        assert log[2] == ("ffn", "rows of mixer", ffn_can and next_takes)


def test_parts_written_before_the_option_existed_are_called_as_before():
    log = []
    mixer = _Part(log, "mixer", False, False, new_style=False)
    ffn = _Part(log, "ffn", False, False, new_style=False)
    block = _block(log, mixer, ffn)
    assert block.forward("x", None, None, h="given", next_norm=None) is None      # no norm asked for: the block runs it later
    assert log == [("mixer", "given", False), ("ffn", "rows of mixer", False)]
    # and the decoder only tells a block about the next layer if the block says it wants to know
    assert PreNormBlock.passes_deferred_rows is True
