"""Per-NVTX-range device time from the SQLite export of an Nsight Systems trace.

    nsys profile -c cudaProfilerApi --export sqlite -o trace python my_script.py     # wherever nsys exists
    python benchmarks/nsys_nvtx_report.py trace.sqlite [--keywords cov_,inv_] [--ignore-first] [--json out.json]

For every NVTX range text: number of calls and mean / standard deviation of (a) the range's own
duration on the host, (b) the device time of the kernels, (c) memsets, (d) memcpys launched from
inside the range and (e) the time spent in synchronisation calls, attributed through the runtime-API
call that launched them (correlation ids), the way the reference's
examples/prof/parse_nvtx_events.py:28-111 does it.  One grouped query per activity table instead
of one query per range occurrence; needs only the standard library.  Ranges of this library that a
trace will show: ``forward_and_backward``, ``update_curvature``, ``update_preconditioner``,
``precondition``, ``cov_kron_A`` / ``cov_kron_B``, ``inv_<shape>_<module>``, ``kfac_curvature`` /
``kfac_inverse`` / ``kfac_precondition``, ``reduce_scatter_curvature``, ``all_gather_grad`` ...

Without an external profiler the same per-range table (device time by CUDA events) comes from
``asdl_b200.utils.PhaseProfile``.
"""
import argparse
import json
import math
import sqlite3

ACTIVITY_TABLES = {'kernel': 'CUPTI_ACTIVITY_KIND_KERNEL', 'memset': 'CUPTI_ACTIVITY_KIND_MEMSET',
                   'memcpy': 'CUPTI_ACTIVITY_KIND_MEMCPY', 'sync': 'CUPTI_ACTIVITY_KIND_SYNCHRONIZATION'}


def _tables(con):
    return {row[0] for row in con.execute("SELECT name FROM sqlite_master WHERE type='table'")}


def _ranges(con, tables):
    """[(range id, text, start, end)]; newer exports keep the text in a string table."""
    columns = {row[1] for row in con.execute('PRAGMA table_info(NVTX_EVENTS)')}
    if 'textId' in columns and 'StringIds' in tables:
        sql = ('SELECT e.rowid, COALESCE(e.text, s.value), e.start, e.end FROM NVTX_EVENTS e '
               'LEFT JOIN StringIds s ON e.textId = s.id WHERE e.end IS NOT NULL')
    else:
        sql = 'SELECT rowid, text, start, end FROM NVTX_EVENTS WHERE end IS NOT NULL'
    return [r for r in con.execute(sql) if r[1] is not None]


def collect(path, keywords=None, texts=None, ignore_first=False):
    """{range text: {'ncalls', 'runtime', 'runtime_stdev', 'kernel', 'kernel_stdev', ...}} in nanoseconds."""
    con = sqlite3.connect(path)
    tables = _tables(con)
    if 'NVTX_EVENTS' not in tables:
        raise ValueError(f'{path} has no NVTX_EVENTS table: was the trace recorded with NVTX enabled?')
    ranges = _ranges(con, tables)
    if texts:
        ranges = [r for r in ranges if r[1] in texts]
    elif keywords:
        ranges = [r for r in ranges if any(k in r[1] for k in keywords)]
    con.execute('CREATE TEMP TABLE wanted (rid INTEGER PRIMARY KEY, text TEXT, start INTEGER, end INTEGER)')
    con.executemany('INSERT INTO wanted VALUES (?, ?, ?, ?)', ranges)
    per_range = {rid: {'text': text, 'start': start, 'runtime': end - start} for rid, text, start, end in ranges}
    for key, table in ACTIVITY_TABLES.items():
        for record in per_range.values():
            record[key] = 0
        if table not in tables or 'CUPTI_ACTIVITY_KIND_RUNTIME' not in tables:
            continue
        sql = (f'SELECT w.rid, SUM(a.end - a.start) FROM wanted w '
               f'JOIN CUPTI_ACTIVITY_KIND_RUNTIME r ON r.start BETWEEN w.start AND w.end '
               f'JOIN {table} a ON a.correlationId = r.correlationId GROUP BY w.rid')
        for rid, total in con.execute(sql):
            per_range[rid][key] = total or 0
    con.close()

    by_text = {}
    for rid in sorted(per_range, key=lambda r: per_range[r]['start']):   # occurrences in time order
        by_text.setdefault(per_range[rid]['text'], []).append(per_range[rid])
    out = {}
    for text, records in by_text.items():
        if ignore_first:
            records = records[1:]
        if not records:
            continue
        row = {'ncalls': len(records)}
        for key in ('runtime', 'kernel', 'memset', 'memcpy', 'sync'):
            values = [r[key] for r in records]
            mean = sum(values) / len(values)
            var = sum((v - mean) ** 2 for v in values) / (len(values) - 1) if len(values) > 1 else 0.0
            row[key], row[key + '_stdev'] = mean, math.sqrt(var)
        out[text] = row
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('sqlite_path')
    ap.add_argument('--texts', default=None, help='comma-separated range names to report (default: all)')
    ap.add_argument('--keywords', default=None, help='comma-separated substrings; ignored when --texts is given')
    ap.add_argument('--ignore-first', action='store_true', help='leave the first occurrence of every range out')
    ap.add_argument('--json', default=None, help='also write the table to this file')
    args = ap.parse_args()
    table = collect(args.sqlite_path, keywords=args.keywords.split(',') if args.keywords else None,
                    texts=set(args.texts.split(',')) if args.texts else None, ignore_first=args.ignore_first)
    width = max([len(t) for t in table] + [5])
    print(f'{"range":<{width}}  {"calls":>6}  {"host ms":>10}  {"kernel ms":>10}  {"memcpy ms":>10}  {"memset ms":>10}  {"sync ms":>10}')
    for text, row in sorted(table.items(), key=lambda kv: -kv[1]['kernel'] * kv[1]['ncalls']):
        print(f'{text:<{width}}  {row["ncalls"]:>6d}  {row["runtime"] / 1e6:>10.4f}  {row["kernel"] / 1e6:>10.4f}  '
              f'{row["memcpy"] / 1e6:>10.4f}  {row["memset"] / 1e6:>10.4f}  {row["sync"] / 1e6:>10.4f}')
    if args.json:
        with open(args.json, 'w') as f:
            json.dump(table, f, indent=1)


if __name__ == '__main__':
    main()
