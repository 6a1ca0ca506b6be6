"""Plain, slow, whole-sequence implementation of the Qwen3 dense decoder.

It rests on the formulas of the reference's Rust sources only (each function
cites file:line, paths relative to the reference project): the reference is
Rust and no Rust toolchain is available where these tests run, so its model
code cannot be imported or compiled and no golden vectors from it exist.

Nothing here imports the product package; the product is compared with this.
"""
