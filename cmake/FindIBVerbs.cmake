# Locates libibverbs. Sets IBVerbs_FOUND, IBVerbs_INCLUDE_DIRS, IBVerbs_LIBRARIES and the target IBVerbs::ibverbs.
# Hints: IBVERBS_ROOT (variable or environment).
find_path(IBVerbs_INCLUDE_DIR NAMES infiniband/verbs.h
          HINTS ${IBVERBS_ROOT} ENV IBVERBS_ROOT PATH_SUFFIXES include
          PATHS /usr /usr/local /opt/mellanox /usr/local/ofed)
find_library(IBVerbs_LIBRARY NAMES ibverbs
             HINTS ${IBVERBS_ROOT} ENV IBVERBS_ROOT PATH_SUFFIXES lib lib64 lib/x86_64-linux-gnu lib/aarch64-linux-gnu
             PATHS /usr /usr/local /opt/mellanox /usr/local/ofed)
include(FindPackageHandleStandardArgs)
find_package_handle_standard_args(IBVerbs DEFAULT_MSG IBVerbs_LIBRARY IBVerbs_INCLUDE_DIR)
if(IBVerbs_FOUND)
  set(IBVerbs_INCLUDE_DIRS ${IBVerbs_INCLUDE_DIR})
  set(IBVerbs_LIBRARIES ${IBVerbs_LIBRARY})
  if(NOT TARGET IBVerbs::ibverbs)
    add_library(IBVerbs::ibverbs UNKNOWN IMPORTED)
    set_target_properties(IBVerbs::ibverbs PROPERTIES IMPORTED_LOCATION "${IBVerbs_LIBRARY}"
                          INTERFACE_INCLUDE_DIRECTORIES "${IBVerbs_INCLUDE_DIR}")
  endif()
endif()
mark_as_advanced(IBVerbs_INCLUDE_DIR IBVerbs_LIBRARY)
