"""Example programs mirroring the reference's `examples/`: every compute kernel as CUDA with a CPU restatement as
oracle and timed baseline. Run any of them with `python -m mojo_b200.examples.<name>`; nothing opens a window."""
