# Locates GDRCopy (gdrapi.h / libgdrapi). Sets GDRCopy_FOUND, GDRCopy_INCLUDE_DIRS, GDRCopy_LIBRARIES and the target
# GDRCopy::gdrapi. Hints: GDRCOPY_ROOT (variable or environment).
find_path(GDRCopy_INCLUDE_DIR NAMES gdrapi.h
          HINTS ${GDRCOPY_ROOT} ENV GDRCOPY_ROOT PATH_SUFFIXES include PATHS /usr /usr/local /opt/gdrcopy)
find_library(GDRCopy_LIBRARY NAMES gdrapi
             HINTS ${GDRCOPY_ROOT} ENV GDRCOPY_ROOT PATH_SUFFIXES lib lib64 lib/x86_64-linux-gnu lib/aarch64-linux-gnu
             PATHS /usr /usr/local /opt/gdrcopy)
include(FindPackageHandleStandardArgs)
find_package_handle_standard_args(GDRCopy DEFAULT_MSG GDRCopy_LIBRARY GDRCopy_INCLUDE_DIR)
if(GDRCopy_FOUND)
  set(GDRCopy_INCLUDE_DIRS ${GDRCopy_INCLUDE_DIR})
  set(GDRCopy_LIBRARIES ${GDRCopy_LIBRARY})
  if(NOT TARGET GDRCopy::gdrapi)
    add_library(GDRCopy::gdrapi UNKNOWN IMPORTED)
    set_target_properties(GDRCopy::gdrapi PROPERTIES IMPORTED_LOCATION "${GDRCopy_LIBRARY}"
                          INTERFACE_INCLUDE_DIRECTORIES "${GDRCopy_INCLUDE_DIR}")
  endif()
endif()
mark_as_advanced(GDRCopy_INCLUDE_DIR GDRCopy_LIBRARY)
