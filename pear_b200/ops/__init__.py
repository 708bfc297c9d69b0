"""Hot ops: fp32 torch statements (:mod:`reference`), sm_100a kernels (:mod:`kernels`, sources in ``csrc/``) and the
dispatching surface the models call (:mod:`api`)."""
