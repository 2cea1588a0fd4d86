"""Shadow tools: a recording mirror in front of an OpenAI-compatible endpoint, a replay of the
recorded requests against a Saber endpoint, and the reader that compares the two.

Parity: `crates/saber-shadow/src/lib.rs:1-10` (mirror / replay / report).
"""
