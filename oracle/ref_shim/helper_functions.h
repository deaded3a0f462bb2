/* TEST INFRASTRUCTURE.  Empty stand-in for the cuda-samples header of the same name
 * (include/utils/utils.h:5); the reference uses nothing from it. */
#pragma once
