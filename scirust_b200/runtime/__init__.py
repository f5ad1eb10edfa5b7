from .raw import (RawAccess, RawBinding, RawBuffer, RawError, RawKernel, RawLaunchConfig, RawRuntime,  # noqa: F401
                  STRICT_IEEE_OPTIONS, compile_cuda_c, validate_alias_groups, validate_launch_geometry)
