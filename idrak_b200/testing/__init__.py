"""What ships for checking a device and an implementation from outside the test tree.

``conformance``  record every operation call of a table of scenarios on the CPU, replay each call on a device, compare
``contracts``    contract suites (fixed cases + seeded random cases) for the pluggable pieces, each with a reference
                 implementation and a deliberately broken twin that the suite must reject
``stress``       long runs, odd shapes, threads; device memory must not grow from step to step
``regression``   save a failing call to a file, replay saved files

Reference: src/Idrak.Abstraction.Testing (Conformance.cs, ContractSuite.cs, Stress.cs, Regression.cs).
"""
from .conformance import CallRecorder, ConformanceReport, RecordedCall, check, record_scenarios, replay  # noqa: F401
from .contracts import ContractSuite, SUITES  # noqa: F401
from .regression import replay_folder, save_case  # noqa: F401
from .stress import StressReport, run_stress  # noqa: F401
