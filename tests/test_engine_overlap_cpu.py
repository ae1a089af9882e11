"""CPU: the driver that advances several decoder passes in turn from one collective to the next."""
import torch

from flash_attn_v100_b200.engine.model import TPDecoder


class _FakeDecoder:
    def __init__(self):
        self.log = []

    def forward_stages(self, name, n_collectives):
        for i in range(n_collectives):
            self.log.append(("compute", name, i))
            yield torch.full((2,), float(i))
        self.log.append(("finish", name))
        return f"hidden-{name}"

    def _all_reduce(self, t):
        self.log.append(("allreduce", float(t[0])))
        return t


def test_passes_are_interleaved_at_their_collectives():
    fake = _FakeDecoder()
    out = TPDecoder.forward_overlapped(fake, [dict(name="a", n_collectives=2), dict(name="b", n_collectives=3)],
                                       [None, None])
    assert out == ["hidden-a", "hidden-b"]
    # a and b alternate: each pass runs up to its next collective, the collective is issued, the other pass follows
    assert fake.log == [
        ("compute", "a", 0), ("allreduce", 0.0), ("compute", "b", 0), ("allreduce", 0.0),
        ("compute", "a", 1), ("allreduce", 1.0), ("compute", "b", 1), ("allreduce", 1.0),
        ("finish", "a"), ("compute", "b", 2), ("allreduce", 2.0),
        ("finish", "b"),
    ]
