"""dense_reader: the decode-time weight-streaming matmul (linear.py) on a B200."""
