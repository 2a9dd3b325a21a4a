# Branch for the reference's top-level CMakeLists.txt, placed beside the "rtx4090-24g" branch
# (CMakeLists.txt:49-84 of the reference).  Same conventions: QINGMING_MODEL_FAMILY picks the family define, the
# production binary is built by one nvcc command from the device directory's main.cu, targets keep their names.
#
#   cmake -DQINGMING_DEVICE=b200-sxm -DQINGMING_MODEL_FAMILY=1.7b -DQM_B200_ROOT=/path/to/this/repository ..
#
# QM_B200_ROOT is the checkout that holds include/qm_attention.h and the built libqm_attention_b200.so.
elseif(QINGMING_DEVICE STREQUAL "b200-sxm")
    set(CUDA_PATH "/usr/local/cuda" CACHE PATH "CUDA Toolkit installation")
    set(NVCC "${CUDA_PATH}/bin/nvcc" CACHE FILEPATH "NVIDIA CUDA compiler")
    set(QM_B200_ROOT "" CACHE PATH "Checkout of the B200 attention path (include/, qingming-qwen3-tts_b200/)")

    if(NOT EXISTS "${NVCC}")
        message(FATAL_ERROR "nvcc not found at ${NVCC}; set CUDA_PATH or NVCC explicitly")
    endif()
    if(NOT EXISTS "${QM_B200_ROOT}/include/qm_attention.h")
        message(FATAL_ERROR "QM_B200_ROOT must point at the checkout that holds include/qm_attention.h")
    endif()

    if(QINGMING_MODEL_FAMILY STREQUAL "1.7b")
        set(FAMILY_DEFINE "QINGMING_MODEL_FAMILY_1_7B=1")
    elseif(QINGMING_MODEL_FAMILY STREQUAL "0.6b")
        set(FAMILY_DEFINE "QINGMING_MODEL_FAMILY_0_6B=1")
    else()
        message(FATAL_ERROR "B200 supports QINGMING_MODEL_FAMILY=0.6b or 1.7b")
    endif()

    set(QM_B200_PACKAGE "${QM_B200_ROOT}/qingming-qwen3-tts_b200")
    set(PROD_NAME "qingming-qwen3-tts_b200-sxm_${QINGMING_MODEL_FAMILY}")
    set(PROD_BINARY "${CMAKE_BINARY_DIR}/${PROD_NAME}")

    add_custom_command(OUTPUT "${PROD_BINARY}"
        COMMAND "${NVCC}" -gencode arch=compute_100a,code=sm_100a "-D${FAMILY_DEFINE}" -std=c++20 -O3 -DNDEBUG
                -Xcompiler=-pthread,-Wall,-Wextra
                -I "${QM_B200_ROOT}/include" -I "${QM_B200_PACKAGE}/host" -I "${QM_B200_PACKAGE}/devices/b200-sxm"
                "${QM_B200_PACKAGE}/devices/b200-sxm/main.cu" -o "${PROD_BINARY}"
                -L "${QM_B200_PACKAGE}/lib" -lqm_attention_b200 "-Xlinker=-rpath=${QM_B200_PACKAGE}/lib"
        DEPENDS "${QM_B200_PACKAGE}/devices/b200-sxm/main.cu" "${QM_B200_PACKAGE}/devices/b200-sxm/device.h"
                "${QM_B200_PACKAGE}/host/talker_engine_b200.hpp" "${QM_B200_PACKAGE}/host/resident_loop_b200.hpp"
                "${QM_B200_PACKAGE}/lib/libqm_attention_b200.so"
        WORKING_DIRECTORY "${CMAKE_SOURCE_DIR}" VERBATIM)
