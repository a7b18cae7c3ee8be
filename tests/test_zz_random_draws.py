"""Random draws built from the uniform fill on the "vulkan" device: torch.bernoulli(p) with a tensor of probabilities,
Tensor.exponential_, F.gumbel_softmax; and pow_ with a tensor exponent. Checked by moments and by reproducibility under a
seed, against the closed forms of the distributions."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vk(cuda):
    import torchvulkan

    assert torchvulkan.is_available() and torchvulkan.device_count() >= 1
    return torch.device("vulkan:0")


def test_bernoulli_of_a_probability_tensor_and_exponential_draws(vk):
    """torch.bernoulli(p) with a tensor of probabilities, Tensor.exponential_ and what is built on them (F.gumbel_softmax):
    checked by their moments, and by reproducibility under a seed."""
    import torchvulkan

    torchvulkan.manual_seed(77)
    p = torch.tensor([0.1, 0.5, 0.9]).repeat(20000, 1)
    draws = torch.bernoulli(p.to(vk)).cpu()
    assert draws.dtype == torch.float32 and set(draws.unique().tolist()) <= {0.0, 1.0}
    assert float((draws.mean(0) - torch.tensor([0.1, 0.5, 0.9])).abs().max()) < 0.015
    mask = torch.empty(20000, 3, dtype=torch.bool, device=vk).bernoulli_(torch.tensor([0.2, 0.4, 0.6]).to(vk)).cpu()
    assert float((mask.float().mean(0) - torch.tensor([0.2, 0.4, 0.6])).abs().max()) < 0.015
    e = torch.empty(60000, device=vk).exponential_(2.0).cpu()
    assert float(e.min()) > 0.0 and bool(torch.isfinite(e).all())
    assert abs(float(e.mean()) - 0.5) < 0.01 and abs(float(e.var()) - 0.25) < 0.02
    torchvulkan.manual_seed(5)
    first = torch.empty(1000, device=vk).exponential_().cpu()
    torchvulkan.manual_seed(5)
    assert torch.equal(torch.empty(1000, device=vk).exponential_().cpu(), first)
    logits = torch.randn(64, 10).to(vk)
    soft = F.gumbel_softmax(logits, tau=0.7).cpu()
    assert float((soft.sum(-1) - 1).abs().max()) < 1e-5 and float(soft.min()) >= 0.0
    hard = F.gumbel_softmax(logits, tau=0.7, hard=True).cpu()
    assert float((hard - hard.round()).abs().max()) < 1e-6 and torch.equal(hard.round().sum(-1), torch.ones(64))      # one-hot up to the rounding of (1 - s) + s
    base = torch.rand(5, 7) + 0.5
    b = base.clone().to(vk)
    b.pow_(torch.full((5, 7), 1.5).to(vk))
    assert torch.allclose(b.cpu(), base.pow(1.5), rtol=1e-5, atol=1e-6)
