# check_blackwell_gpu(<result variable>): compiles and runs a tiny host program that asks the CUDA runtime for the
# devices of this machine; the result is TRUE when at least one has compute capability 10.x. Information only: the
# libraries are always built for sm_100a (nvcc cross-compiles on machines without a GPU). The program makes no
# allocation, launches nothing and changes no device setting.
function(check_blackwell_gpu result)
  set(${result} FALSE PARENT_SCOPE)
  if(NOT CUDAToolkit_FOUND)
    return()
  endif()
  set(src "${CMAKE_CURRENT_FUNCTION_LIST_DIR}/check_blackwell_gpu.cc")
  try_run(run_rc compile_ok "${CMAKE_BINARY_DIR}/check_blackwell_gpu" "${src}"
          CMAKE_FLAGS "-DINCLUDE_DIRECTORIES=${CUDAToolkit_INCLUDE_DIRS}"
          LINK_LIBRARIES CUDA::cudart_static
          RUN_OUTPUT_VARIABLE run_out)
  if(compile_ok AND run_rc EQUAL 0)
    set(${result} TRUE PARENT_SCOPE)
    message(STATUS "Blackwell GPU found: ${run_out}")
  else()
    message(STATUS "No Blackwell (sm_100) GPU visible at configure time; building for sm_100a anyway")
  endif()
endfunction()
