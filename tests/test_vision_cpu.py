import torch

from pear_b200.models.vision import VisionConfig, VisionTower


def test_vision_tower_shapes_grouping_and_isolation():
    cfg = VisionConfig.tiny(out_hidden=32)
    tower = VisionTower(cfg).init_weights(1)
    a, b, c = torch.randn(3, 16, 16), torch.randn(3, 32, 16), torch.randn(3, 16, 16)
    out = tower([a, b, c])
    assert [tuple(o.shape) for o in out] == [(4, 32), (8, 32), (4, 32)] and tower.tokens_per_image(32, 16) == 8
    # an image's rows do not depend on what else is in the batch (attention never crosses images)
    alone = tower([c])[0]
    assert torch.allclose(out[2], alone, atol=1e-5)
    out[0].sum().backward()
    assert tower.patch_embed.weight.grad is not None
