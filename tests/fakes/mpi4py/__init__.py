"""A stand-in for mpi4py, for tests only: the few calls that ``iris_b200.parallel.bootstrap.MpiBootstrap`` makes,
implemented over a ``torch.distributed.FileStore`` (rank and size come from the launcher's environment, as they do from
``mpirun``).  mpi4py itself is not installed on the test machines; this lets the MPI code path of the bootstrap run as
real processes.  The real module's semantics that matter here are kept: collectives are matched by call order, and
``Ibarrier`` returns a request whose ``Test()`` turns true once every rank has entered."""
