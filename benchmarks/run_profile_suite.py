"""Run the automated profiler over a workload list and write BOTH report formats into one folder.

Counterpart of the reference's ``scripts/run_profile_suite.py``: ``<output-dir>/<prefix>.json`` (full
report) and ``<output-dir>/<prefix>.csv`` (appended rows), then the summary table.

    python benchmarks/run_profile_suite.py --output-dir reports --workloads logp_fused,sampling_fused
    python benchmarks/run_profile_suite.py --smoke --device cpu --output-dir /tmp/reports
"""

import sys
from datetime import datetime, timezone
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

import profiler as prof  # noqa: E402


def build_script_parser():
    """The profiler's own command line plus the flags that say where the two report files go."""
    parser = prof.build_arg_parser()
    parser.add_argument("--output-dir", type=Path, default=Path("profile_reports"))
    parser.add_argument("--prefix", default=None, help="report file stem (default: profile_<UTC timestamp>)")
    parser.add_argument("--fail-on-blocked", action="store_true", help="exit 1 when any workload was blocked")
    return parser


def main() -> None:
    args = build_script_parser().parse_args()
    if args.smoke:
        args.dtype, args.warmup, args.repeat, args.hidden = "float32", 0, 1, 16
    stem = args.prefix or datetime.now(timezone.utc).strftime("profile_%Y%m%dT%H%M%SZ")
    suite = prof.run_automated_suite(args)
    suite.save_json(args.output_dir / f"{stem}.json")
    suite.save_csv(args.output_dir / f"{stem}.csv")
    if not args.no_summary:
        suite.print_summary()
    blocked = [m.benchmark_name for m in suite.get_metrics() if m.status != "pass"]
    print(f"reports: {args.output_dir / (stem + '.json')}  {args.output_dir / (stem + '.csv')}  blocked: {blocked or 'none'}")
    if blocked and args.fail_on_blocked:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
