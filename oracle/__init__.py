"""CPU oracle for the dense_reader path: test infrastructure only (see oracle.c's header). Never imported by the
product package."""
