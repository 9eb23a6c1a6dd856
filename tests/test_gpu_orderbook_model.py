"""The order-book transformer (dilated sparse attention inside a pre-LN block):
bf16 forward on the native kernels against the same network in fp32 torch with a
dense masked attention."""
import pytest
import torch

from ma_transformer_b200 import _native as nat
from ma_transformer_b200.layers.orderbook_model import OrderBookTransformer, synthetic_ticks
from helpers import orderbook_reference_forward as reference_forward

pytestmark = pytest.mark.gpu


def test_orderbook_forward_matches_fp32_reference():
    torch.manual_seed(0)
    model = OrderBookTransformer().eval()
    ticks = synthetic_ticks(2, 512, seed=1)
    ticks = (ticks - ticks.mean(dim=(0, 1))) / (ticks.std(dim=(0, 1)) + 1e-6)   # feature scaling, as a loader would
    with torch.no_grad():
        want = reference_forward(model, ticks)
        got32 = model.cuda()(ticks.cuda())
        assert nat.last_kernel() == "mma_window_f32"                            # fp32: three TF32 products per product
        got16 = model.to(torch.bfloat16)(ticks.cuda().to(torch.bfloat16))
        assert nat.last_kernel() == "umma_band"                                 # bf16: the tcgen05 band kernel
    assert got32.shape == (2, 3)
    assert (got32.cpu() - want).abs().max() <= 2e-3 * max(1.0, float(want.abs().max()))
    # bf16 weights and activations through 4 layers: compare loosely, relative to the logits' scale
    assert (got16.float().cpu() - want).abs().max() <= 0.08 * max(1.0, float(want.abs().max()))


def test_synthetic_ticks_shape_and_book_order():
    t = synthetic_ticks(3, 100, seed=2)
    assert t.shape == (3, 100, 40)
    bid, ask, sizes = t[..., :10], t[..., 10:20], t[..., 20:]
    assert (ask > bid).all() and (bid[..., 0] > bid[..., 9]).all() and (sizes > 0).all()
