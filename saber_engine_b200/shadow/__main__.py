"""`python -m saber_engine_b200.shadow mirror|replay|report`.  Nothing here reads the environment:
the log directory, the upstream and the target are arguments.

Parity: `crates/saber-shadow/src/main.rs`.
"""
import argparse
import asyncio
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="saber-shadow")
    sub = ap.add_subparsers(dest="cmd", required=True)
    m = sub.add_parser("mirror", help="recording reverse proxy in front of an OpenAI-compatible endpoint")
    m.add_argument("--upstream", required=True)
    m.add_argument("--log-dir", required=True)
    m.add_argument("--host", default="127.0.0.1")
    m.add_argument("--port", type=int, default=8081)
    p = sub.add_parser("replay", help="send a day's recorded requests to a Saber endpoint")
    p.add_argument("--log", required=True)
    p.add_argument("--target", required=True)
    p.add_argument("--out", required=True)
    p.add_argument("--pace", default="sequential", choices=["sequential", "recorded"])
    p.add_argument("--speed", type=float, default=1.0)
    p.add_argument("--api-key", default=None)
    r = sub.add_parser("report", help="compare a mirror log with a replay file; exit 1 when a stop fired")
    r.add_argument("--log", required=True)
    r.add_argument("--replay", required=True)
    r.add_argument("--engine-log", default=None)
    r.add_argument("--power-w", type=float, default=1000.0)
    a = ap.parse_args(argv)
    if a.cmd == "mirror":
        import uvicorn
        from .mirror import Mirror
        uvicorn.run(Mirror(a.upstream, a.log_dir).app(), host=a.host, port=a.port, log_level="warning")
        return 0
    if a.cmd == "replay":
        from .replay import replay
        print(asyncio.run(replay(a.log, a.target, a.out, a.pace, a.speed, a.api_key)))
        return 0
    from .report import read
    rep = read(a.log, a.replay, open(a.engine_log).read() if a.engine_log else None, expect_power_w=a.power_w)
    print(rep.render())
    return 1 if rep.fired else 0


if __name__ == "__main__":
    sys.exit(main())
