"""The synthetic-layer packers of the package write the engine's layouts: byte for byte the oracle's packers (which
tests/test_oracle_pins.py pins to the reference's)."""
import numpy as np


def test_synth_packers_equal_oracle_packers(orc):
    import torch
    from dsgx10_b200 import synth
    rng = np.random.default_rng(3)
    q = rng.integers(0, 256, (32, 512), dtype=np.uint8)
    assert (synth.tile_fp8(torch.from_numpy(q)).numpy() == orc.pack_fp8_tile(q)).all()
    assert (synth.untile_fp8(synth.tile_fp8(torch.from_numpy(q)), 32, 512).numpy() == q).all()
    wp, s = synth.int4_tensors(16, 1024, 5)
    assert (synth.pack_int4_block(wp, s) == orc.pack_int4_block(wp, s, None)).all()
    wb = rng.integers(0, 65536, (16, 256), dtype=np.uint16)
    assert (synth.tile_bf16(wb) == orc.pack_bf16_tile(wb)).all()


def test_fp8_weight_quantisation_rule(orc):
    """scale = amax / 448 per 128x128 block, codes = e4m3(w / scale): every block's largest code is +-448."""
    import torch
    from dsgx10_b200 import synth
    w = torch.randn(256, 384, generator=torch.Generator().manual_seed(1)) * 0.02
    q, s = synth.quant_fp8_128(w)
    deq = orc.e4m3_to_f32(q.numpy()).reshape(2, 128, 3, 128) * s.numpy()[:, None, :, None]
    assert np.abs(deq.reshape(256, 384) - w.numpy()).max() <= 0.0625 * np.abs(w.numpy()).max()
    assert (np.abs(orc.e4m3_to_f32(q.numpy())).reshape(2, 128, 3, 128).max(axis=(1, 3)) == 448).all()
