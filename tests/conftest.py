"""Shared fixtures.  Tests that need a GPU carry ``@pytest.mark.gpu``; everything else runs on CPU
(multi-process tests use the gloo backend)."""
import os
import sys

import pytest
import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: test needs a CUDA device (B200)')


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)


def make_mlp(in_dim=5, hid_dim=4, out_dim=3, bias=True):
    return nn.Sequential(nn.Linear(in_dim, hid_dim, bias=bias), nn.ReLU(),
                         nn.Linear(hid_dim, hid_dim, bias=bias), nn.ReLU(),
                         nn.Linear(hid_dim, out_dim, bias=bias))


def make_cnn(in_dim=5, hid_dim=4, out_dim=3):
    return nn.Sequential(nn.Conv2d(in_dim, hid_dim, kernel_size=2), nn.ReLU(),
                         nn.Conv2d(hid_dim, hid_dim, kernel_size=2), nn.ReLU(),
                         nn.Flatten(), nn.Linear(hid_dim * 2 * 2, out_dim))


def make_net(kind, **kw):
    torch.manual_seed(1)
    return make_mlp(**kw) if kind == 'mlp' else make_cnn(**kw)


def make_data(kind, n, loss_type, in_dim=5, out_dim=3, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, in_dim, generator=g) if kind == 'mlp' else torch.randn(n, in_dim, 4, 4, generator=g)
    if loss_type == 'cross_entropy':
        t = torch.randint(out_dim, (n,), generator=g)
    else:
        t = torch.randn(n, out_dim, generator=g)
    return x, t


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(1234)
    yield
