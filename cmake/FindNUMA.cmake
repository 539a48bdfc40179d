# Locates libnuma. Sets NUMA_FOUND, NUMA_INCLUDE_DIRS, NUMA_LIBRARIES and the target NUMA::numa.
# Hints: NUMA_ROOT (variable or environment). The library binds its proxy threads with sched_setaffinity and reads the
# GPU's NUMA node from sysfs (csrc/core/numa.cc), so libnuma is optional.
find_path(NUMA_INCLUDE_DIR NAMES numa.h HINTS ${NUMA_ROOT} ENV NUMA_ROOT PATH_SUFFIXES include PATHS /usr /usr/local)
find_library(NUMA_LIBRARY NAMES numa
             HINTS ${NUMA_ROOT} ENV NUMA_ROOT PATH_SUFFIXES lib lib64 lib/x86_64-linux-gnu lib/aarch64-linux-gnu
             PATHS /usr /usr/local)
include(FindPackageHandleStandardArgs)
find_package_handle_standard_args(NUMA DEFAULT_MSG NUMA_LIBRARY NUMA_INCLUDE_DIR)
if(NUMA_FOUND)
  set(NUMA_INCLUDE_DIRS ${NUMA_INCLUDE_DIR})
  set(NUMA_LIBRARIES ${NUMA_LIBRARY})
  if(NOT TARGET NUMA::numa)
    add_library(NUMA::numa UNKNOWN IMPORTED)
    set_target_properties(NUMA::numa PROPERTIES IMPORTED_LOCATION "${NUMA_LIBRARY}" INTERFACE_INCLUDE_DIRECTORIES "${NUMA_INCLUDE_DIR}")
  endif()
endif()
mark_as_advanced(NUMA_INCLUDE_DIR NUMA_LIBRARY)
