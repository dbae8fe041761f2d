"""Bar charts of the two report formats of this folder, as text (always) and as PNG files (when
matplotlib is installed).

    python benchmarks/time_step.py --optim kfac --model resnet18 --json > kfac.json
    python benchmarks/time_step.py --optim shampoo --model resnet18 --json > shampoo.json
    python benchmarks/plot_report.py phases kfac.json shampoo.json [--png phases.png]

    python benchmarks/flops_memory.py --model resnet50 --json r50.json
    python benchmarks/plot_report.py cost r50.json [--png cost.png]

``phases``: one stacked bar per run, the step split into forward_and_backward / update_curvature /
update_preconditioner / precondition / optimizer_step (mean milliseconds per step, the rest of the
step as "other").  ``cost``: floating-point operations and stored numbers per phase and method.
Role of the reference's examples/prof/plot_rt_cuda.py and plot_flops_memory*.py.
"""
import argparse
import json

PHASES = ['forward_and_backward', 'update_curvature', 'update_preconditioner', 'precondition', 'optimizer_step']
METHODS = {'SGD': ['Forward', 'BackwardWeight', 'BackwardInput'], 'Adam': ['AdamStats', 'AdamPrecond'],
           'K-FAC': ['KFACStats', 'KFACInv', 'KFACPrecond'], 'Shampoo': ['ShampooStats', 'ShampooInv', 'ShampooPrecond'],
           'L-BFGS': ['LBFGSPrecond'], 'SMW-NG': ['SMWNGStats', 'SMWNGPrecond']}


def _last_json_line(path):
    with open(path) as f:
        text = f.read().strip()
    try:
        return json.loads(text)
    except json.JSONDecodeError:
        return json.loads(text.splitlines()[-1])


def phase_rows(paths):
    """[(label, {phase: ms per step})] with per-step means: a phase that runs every k-th step counts 1/k."""
    rows = []
    for path in paths:
        rec = _last_json_line(path)
        ranges = rec['ranges']
        steps = ranges['step']['ncalls']
        parts = {p: ranges[p]['total_ms'] / steps for p in PHASES if p in ranges}
        parts['other'] = max(ranges['step']['total_ms'] / steps - sum(parts.values()), 0.0)
        rows.append((f"{rec.get('optim', '?')} / {rec.get('model', '?')}", parts))
    return rows


def text_bars(rows, unit, width=60):
    """One line per (label, {part: value}): parts as runs of distinct letters scaled to the largest total."""
    fixed = {'forward_and_backward': 'F', 'update_curvature': 'C', 'update_preconditioner': 'U', 'precondition': 'P',
             'optimizer_step': 'O', 'other': '.'}
    names = []
    for _, parts in rows:
        names += [n for n in parts if n not in names]
    spare = iter('abcdefghijklmnopqrstuvwxyz')
    letters = [fixed.get(n) or next(spare) for n in names]
    top = max(sum(parts.values()) for _, parts in rows) or 1.0
    pad = max(len(label) for label, _ in rows)
    lines = ['legend: ' + ', '.join(f'{letters[i]}={n}' for i, n in enumerate(names))]
    for label, parts in rows:
        bar = ''.join(letters[names.index(n)] * round(width * v / top) for n, v in parts.items())
        lines.append(f'{label:<{pad}} |{bar:<{width}}| {sum(parts.values()):.4g} {unit}')
    return '\n'.join(lines)


def cost_rows(path, key):
    rec = _last_json_line(path)
    rows = []
    for method, phases in METHODS.items():
        parts = {p: rec['phases'][p][key] for p in phases if p in rec['phases']}
        if parts:
            rows.append((method, parts))
    return rows


def save_png(rows, unit, path):
    import matplotlib
    matplotlib.use('Agg')
    import matplotlib.pyplot as plt
    fig, ax = plt.subplots(figsize=(1.6 * len(rows) + 2, 4))
    names = []
    for _, parts in rows:
        names += [n for n in parts if n not in names]
    bottoms = [0.0] * len(rows)
    for name in names:
        values = [parts.get(name, 0.0) for _, parts in rows]
        ax.bar(range(len(rows)), values, bottom=bottoms, label=name)
        bottoms = [b + v for b, v in zip(bottoms, values)]
    ax.set_xticks(range(len(rows)))
    ax.set_xticklabels([label for label, _ in rows], rotation=20, ha='right')
    ax.set_ylabel(unit)
    ax.legend(fontsize=7)
    fig.tight_layout()
    fig.savefig(path, dpi=150)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('kind', choices=['phases', 'cost'])
    ap.add_argument('files', nargs='+')
    ap.add_argument('--png', default=None)
    args = ap.parse_args()
    if args.kind == 'phases':
        charts = [(phase_rows(args.files), 'ms / step')]
    else:
        charts = [(cost_rows(args.files[0], 'flop'), 'FLOP'), (cost_rows(args.files[0], 'numel'), 'stored numbers')]
    for i, (rows, unit) in enumerate(charts):
        print(text_bars(rows, unit))
        if args.png:
            try:
                save_png(rows, unit, args.png if i == 0 else args.png.replace('.png', f'_{i}.png'))
            except ImportError:
                print('matplotlib is not installed: text chart only')


if __name__ == '__main__':
    main()
