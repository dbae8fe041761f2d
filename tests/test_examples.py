"""The example scripts and the analytic cost report run end to end on CPU (short settings)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=600):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES='')
    result = subprocess.run([sys.executable, *args], cwd=ROOT, capture_output=True, text=True, timeout=timeout, env=env)
    assert result.returncode == 0, result.stderr[-2000:]
    return result.stdout


@pytest.mark.parametrize('optim', ['kfac_fused', 'shampoo', 'kron_psgd', 'kbfgs', 'ekfac'])
def test_train_script_with_every_family(optim):
    out = _run('examples/train.py', '--optim', optim, '--model', 'cnn', '--steps-per-epoch', '3', '--epochs', '1',
               '--batch-size', '16', '--lr', '0.01', '--no-cuda')
    assert 'avg_step_time' in out and 'nan' not in out.lower()


def test_train_script_reads_json_config():
    out = _run('examples/train.py', '--config', 'examples/configs/cnn_shampoo.json', '--steps-per-epoch', '2',
               '--epochs', '1', '--no-cuda')
    assert 'epoch 1' in out


def test_other_examples():
    assert 'top 2 eigenvalues' in _run('examples/spectrum.py', '--top-n', '2')
    assert 'reshape' in _run('examples/grad_maker_demo.py')
    assert 'epoch 1' in _run('examples/pseudo_batch_train.py', '--epochs', '1')
    assert 'GFLOP' in _run('benchmarks/flops_memory.py', '--model', 'resnet_tiny')


@pytest.mark.parametrize('impl', ['ours', 'fused'])
def test_cpu_mlp_kfac_benchmark_matches_dense_oracle(impl):
    import json
    rec = json.loads(_run('benchmarks/cpu_mlp_kfac.py', '--impl', impl, '--steps', '2').strip().splitlines()[-1])
    assert rec['max_rel_err_vs_dense_oracle'] < 1e-5
    assert rec['last_loss'] < rec['first_loss']
