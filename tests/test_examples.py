"""The example scripts and the analytic cost report run end to end on CPU (short settings)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run_process(*args, timeout=600):
    """The script as its own process (what a user types)."""
    env = dict(os.environ, CUDA_VISIBLE_DEVICES='')
    result = subprocess.run([sys.executable, *args], cwd=ROOT, capture_output=True, text=True, timeout=timeout, env=env)
    assert result.returncode == 0, result.stderr[-2000:]
    return result.stdout


def _run(script, *args):
    """The script's ``__main__`` inside this process (saves an interpreter start and a torch import per
    call); returns what it printed."""
    import contextlib
    import io
    import runpy
    import torch
    out = io.StringIO()
    old_argv, old_path, old_cwd, rng = sys.argv, list(sys.path), os.getcwd(), torch.get_rng_state()
    sys.argv = [os.path.join(ROOT, script), *map(str, args)]
    os.chdir(ROOT)
    try:
        with contextlib.redirect_stdout(out):
            try:
                runpy.run_path(sys.argv[0], run_name='__main__')
            except SystemExit as exc:
                assert exc.code in (None, 0), f'{script} exited with {exc.code}: {out.getvalue()[-2000:]}'
    finally:
        sys.argv, sys.path[:] = old_argv, old_path
        os.chdir(old_cwd)
        torch.set_rng_state(rng)
        for name in ('train', 'augment'):     # modules the scripts import from their own folder
            sys.modules.pop(name, None)
    return out.getvalue()


@pytest.mark.parametrize('optim', ['kfac_fused', 'shampoo', 'kron_psgd', 'kbfgs', 'ekfac'])
def test_train_script_with_every_family(optim):
    out = _run('examples/train.py', '--optim', optim, '--model', 'cnn', '--steps-per-epoch', '3', '--epochs', '1',
               '--batch-size', '16', '--lr', '0.01', '--no-cuda')
    assert 'avg_step_time' in out and 'nan' not in out.lower()


def test_train_script_reads_json_config():
    out = _run_process('examples/train.py', '--config', 'examples/configs/cnn_shampoo.json', '--steps-per-epoch', '2',
               '--epochs', '1', '--no-cuda')
    assert 'epoch 1' in out


def test_other_examples():
    assert 'top 2 eigenvalues' in _run('examples/spectrum.py', '--top-n', '2')
    assert 'reshape' in _run('examples/grad_maker_demo.py')
    assert 'epoch 1' in _run('examples/pseudo_batch_train.py', '--epochs', '1')
    assert 'GFLOP' in _run('benchmarks/flops_memory.py', '--model', 'resnet_tiny')
    assert 'K-FAC OBS pruning' in _run('examples/one_shot_pruning.py', '--rounds', '2')


@pytest.mark.parametrize('impl', ['ours', 'fused'])
def test_cpu_mlp_kfac_benchmark_matches_dense_oracle(impl):
    import json
    rec = json.loads(_run('benchmarks/cpu_mlp_kfac.py', '--impl', impl, '--steps', '2').strip().splitlines()[-1])
    assert rec['max_rel_err_vs_dense_oracle'] < 1e-5
    assert rec['last_loss'] < rec['first_loss']


def test_batched_augmentations_match_per_sample_definitions():
    import torch
    import torch.nn.functional as F
    sys.path.insert(0, os.path.join(ROOT, 'examples'))
    from augment import batch_cutout, batch_random_crop_flip, Cutout
    x = torch.randn(6, 3, 8, 8)
    g = torch.Generator().manual_seed(3)
    out = batch_random_crop_flip(x, padding=2, generator=g)
    g = torch.Generator().manual_seed(3)   # replay the draws: dy, dx, then the flip coin
    dy = torch.randint(-2, 3, (6, 1, 1), generator=g).flatten()
    dx = torch.randint(-2, 3, (6, 1, 1), generator=g).flatten()
    flip = (torch.rand(6, 1, 1, generator=g) < 0.5).flatten()
    for i in range(6):
        padded = F.pad(x[i], (2, 2, 2, 2))
        crop = padded[:, 2 + dy[i]:2 + dy[i] + 8, 2 + dx[i]:2 + dx[i] + 8]
        want = crop.flip(-1) if flip[i] else crop
        torch.testing.assert_close(out[i], want)
    holes = batch_cutout(torch.ones(5, 2, 16, 16), n_holes=1, length=4, generator=torch.Generator().manual_seed(0))
    zeros = (holes[:, 0] == 0).flatten(1).sum(dim=1)
    assert ((zeros > 0) & (zeros <= 16)).all() and torch.equal(holes[:, 0], holes[:, 1])
    assert Cutout(2, 4)(torch.ones(3, 16, 16)).shape == (3, 16, 16)


def test_train_script_accepts_reference_style_config(tmp_path):
    import json
    cfg = {'dataset': 'synthetic', 'model': 'resnet18', 'optim': 'kfac_mc', 'lr': 0.01, 'momentum': 0.9, 'damping': 1e-3,
           'curvature_update_interval': 2, 'clipping_norm': 10, 'ema_decay': -1, 'data_augmentation': True, 'cutout': True,
           'n_holes': 1, 'length': 16, 'batch_size': 8, 'epochs': 1, 'weight_decay': 5e-4}
    path = tmp_path / 'cfg.json'
    path.write_text(json.dumps(cfg))
    log = tmp_path / 'log.jsonl'
    out = _run('examples/train.py', '--config', str(path), '--steps-per-epoch', '3', '--no-cuda', '--cosine',
               '--label-smoothing', '0.1', '--log-json', str(log))
    assert 'epoch 1' in out
    lines = [json.loads(line) for line in log.read_text().splitlines()]
    assert lines[0]['epoch'] == 1 and 'avg_step_time_ms' in lines[-1] and lines[-1]['stopped'] is None


def test_every_recipe_parses_and_builds_its_maker(monkeypatch):
    """All entries of examples/configs/recipes.json name valid options, models and methods."""
    import json
    sys.path.insert(0, os.path.join(ROOT, 'examples'))
    import train
    with open(os.path.join(ROOT, 'examples', 'configs', 'recipes.json')) as f:
        table = json.load(f)
    count = 0
    for family, entries in table.items():
        if family.startswith('_'):
            continue
        for method in entries:
            if method == 'common':
                continue
            monkeypatch.setattr(sys, 'argv', ['train.py', '--recipe', f'{family}/{method}', '--dataset', 'synthetic',
                                              '--batch-size', '4', '--no-cuda'])
            args = train.parse_args()
            assert args.dataset == 'synthetic' and args.batch_size == 4 and args.optim in train.OPTIMS
            assert args.preconditioner_upd_interval == args.curvature_upd_interval
            if family in ('mlp', 'resnet18'):   # the big families are built in the model tests
                model = train.make_model(args.model, (3, 32, 32), 10, 32, args.depth)
                assert train.make_grad_maker(args, model) is not None
            count += 1
    assert count == 25


def test_recipe_runs_end_to_end():
    out = _run('examples/train.py', '--recipe', 'mlp/kfac', '--dataset', 'synthetic', '--width', '32', '--batch-size', '8',
               '--steps-per-epoch', '3', '--epochs', '1', '--no-cuda')
    assert 'epoch 1' in out


def test_nsys_report_attributes_kernels_to_ranges(tmp_path):
    """A hand-made export: two occurrences of range 'cov' with kernels of 30 + 20 and 50 ns launched
    inside them, one 'inv' range with a memcpy, and a kernel launched outside every range."""
    import sqlite3
    sys.path.insert(0, os.path.join(ROOT, 'benchmarks'))
    import nsys_nvtx_report as report
    db = str(tmp_path / 'trace.sqlite')
    con = sqlite3.connect(db)
    con.execute('CREATE TABLE NVTX_EVENTS (start INTEGER, end INTEGER, text TEXT)')
    con.executemany('INSERT INTO NVTX_EVENTS VALUES (?, ?, ?)', [(100, 200, 'cov'), (300, 420, 'cov'), (500, 600, 'inv'),
                                                                 (700, None, 'open')])
    con.execute('CREATE TABLE CUPTI_ACTIVITY_KIND_RUNTIME (start INTEGER, end INTEGER, correlationId INTEGER)')
    con.executemany('INSERT INTO CUPTI_ACTIVITY_KIND_RUNTIME VALUES (?, ?, ?)',
                    [(110, 115, 1), (150, 155, 2), (310, 315, 3), (510, 515, 4), (650, 655, 5)])
    con.execute('CREATE TABLE CUPTI_ACTIVITY_KIND_KERNEL (start INTEGER, end INTEGER, correlationId INTEGER)')
    con.executemany('INSERT INTO CUPTI_ACTIVITY_KIND_KERNEL VALUES (?, ?, ?)',
                    [(1000, 1030, 1), (1030, 1050, 2), (1100, 1150, 3), (1300, 1400, 5)])
    con.execute('CREATE TABLE CUPTI_ACTIVITY_KIND_MEMCPY (start INTEGER, end INTEGER, correlationId INTEGER)')
    con.execute('INSERT INTO CUPTI_ACTIVITY_KIND_MEMCPY VALUES (1200, 1207, 4)')
    con.commit()
    con.close()
    table = report.collect(db)
    assert set(table) == {'cov', 'inv'}
    assert table['cov']['ncalls'] == 2 and table['cov']['kernel'] == 50 and table['cov']['runtime'] == 110
    assert table['cov']['kernel_stdev'] == 0 and abs(table['cov']['runtime_stdev'] - 200 ** 0.5) < 1e-9
    assert table['inv']['kernel'] == 0 and table['inv']['memcpy'] == 7 and table['inv']['sync'] == 0
    assert report.collect(db, ignore_first=True)['cov']['ncalls'] == 1
    assert set(report.collect(db, keywords=['in'])) == {'inv'}
    assert 'cov' in _run('benchmarks/nsys_nvtx_report.py', db, '--json', str(tmp_path / 'out.json'))


def test_time_step_reports_phases(tmp_path):
    import json
    cfg = tmp_path / 'cfg.yaml'
    cfg.write_text('optim: kfac\nmodel: cnn\nbatch_size: 8\nema_decay: 0.1\niters: 3\nwarmup: 1\n')
    out = _run('benchmarks/time_step.py', '--config', str(cfg), '--no-cuda', '--json')
    ranges = json.loads(out.strip().splitlines()[-1])['ranges']
    assert ranges['step']['ncalls'] == 3 and ranges['optimizer_step']['ncalls'] == 3
    assert ranges['step']['mean_ms'] >= ranges['update_curvature']['mean_ms'] > 0
    assert 'cov_kron_A' in ranges and 'precondition' in ranges


def test_api_reference_is_current(tmp_path):
    """docs/api.md is what docs/build_api.py writes from the present docstrings, and every public
    class and function has a docstring."""
    import inspect
    import asdl_b200
    missing = [n for n in dir(asdl_b200) if not n.startswith('_')
               and (inspect.isclass(getattr(asdl_b200, n)) or inspect.isfunction(getattr(asdl_b200, n)))
               and not (getattr(asdl_b200, n).__doc__ or '').strip()]
    assert not missing, missing
    path = os.path.join(ROOT, 'docs', 'api.md')
    with open(path) as f:
        before = f.read()
    try:
        _run('docs/build_api.py')
        with open(path) as f:
            after = f.read()
    finally:
        with open(path, 'w') as f:
            f.write(before)
    assert before == after, 'run python docs/build_api.py'


def test_plot_report_renders_both_formats(tmp_path):
    phases = tmp_path / 'phases.json'
    phases.write_text(_run('benchmarks/time_step.py', '--optim', 'kfac', '--model', 'cnn', '--batch-size', '8',
                           '--iters', '2', '--warmup', '1', '--no-cuda', '--json'))
    out = _run('benchmarks/plot_report.py', 'phases', str(phases))
    assert 'kfac / cnn' in out and 'C=update_curvature' in out and 'ms / step' in out
    cost = tmp_path / 'cost.json'
    _run('benchmarks/flops_memory.py', '--model', 'resnet_tiny', '--json', str(cost))
    out = _run('benchmarks/plot_report.py', 'cost', str(cost))
    assert 'K-FAC' in out and 'Shampoo' in out and 'stored numbers' in out


def test_resnet50_example_loop_on_cpu():
    out = _run('examples/train_resnet50_with_kfac.py', '--cpu-smoke', '--steps', '8', '--batch-size', '4',
               '--cov-update-freq', '2', '--inv-update-freq', '4', '--warmup-steps', '3')
    assert 'step 8/8' in out and 'nan' not in out.lower()
