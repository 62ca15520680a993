"""Test oracle of the optimizer path: CPU restatement (oracle.c) and the reference's own CUDA backend built into
oracle/_ref/. Test infrastructure only: the product package never imports this."""
